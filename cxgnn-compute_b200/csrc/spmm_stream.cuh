// Interface between cxg_spmm_csr and its edge-tiled streaming path (spmm_stream.cu).
#pragma once
#include "common.cuh"

namespace cxg {

// Header words of the streaming workspace.
enum { kSHdrNumLong = 0, kSHdrNumBlocks = 1, kSHdrError = 63 };  // word 63 is the error word of every SpMM workspace header
// Values of the error word.
enum { kSErrNone = 0, kSErrTimeout = 1, kSErrEdgeCount = 2 };
// Row fetch variants: 16-byte async copies into shared memory (default), one bulk
// async copy per row into shared memory.
enum { kModeCpAsync = 0, kModeBulk = 1 };
// Bytes of one chunk of the id ring of the lean walk (two chunks per warp).
constexpr int kIdxChunkBytes = 512;

struct StreamArgs {
  const void *ptr;
  const void *idx;
  const void *x;
  void *y;
  const float *edge_val;
  const int32_t *edge_rel;
  const int64_t *targets;
  int64_t n_dst;
  int64_t nnz;  // edges the caller declared: the workspace is sized for them, no kernel goes beyond
  int64_t rel_stride;
  int64_t max_tiles;
  long long wait_cycles;  // limit of one mbarrier wait (bulk-copy variant)
  int test_stall;         // test hook: the first stage of tile 0 announces bytes that never arrive
  int width, feat, heads, ptr_bytes, reduce, accumulate;
  int tile;         // edges per tile
  int stage_edges;  // edges per ring stage
  int stage_bytes;  // stage_edges * row bytes
  int slot_offset;  // offset of the row slots inside a warp's shared memory
  int warp_smem;    // shared memory per warp
  int max_long;
  int max_blocks;
  int cpr_shift;  // log2(16-byte chunks per row), -1 when not a power of two
  int mode;       // how feature rows are fetched: kModeCpAsync / kModeBulk
  int tma_index;  // lean walk: source ids staged by bulk copies into a ring in shared memory
  int32_t *hdr;
  int64_t *tile_row;    // row that owns the first edge of each tile
  int64_t *tail_row;    // row left unfinished at the end of each tile, or -1
  int64_t *long_tiles;  // tiles whose unfinished row spans more than 64 tiles
  int32_t *long_base;   // first entry of each such chain in the block table
  int32_t *block_owner; // block table: the chain (slot of long_tiles) every block of 64 partials belongs to
  float *block_sums;    // [block][width]: sum of a block's partials
  float *partials;      // [tile][2][width]: head partial, tail partial
};

struct StreamLayout {
  size_t hdr, tile_row, tail_row, long_tiles, long_base, block_owner, block_sums, partials, total;
  int64_t max_tiles;
  int max_long, max_blocks;
};

// True when the descriptor can take the streaming path (16-byte rows up to 1 KiB, no edge mask).
bool stream_eligible(const cxg_spmm_desc *d);
// Edges per tile for this call (desc->split_edges when set).
int stream_tile_edges(const cxg_spmm_desc *d);
int stream_layout(int64_t nnz, int64_t width, int tile, StreamLayout *L);
int stream_launch(const cxg_spmm_desc *d, void *workspace, size_t workspace_bytes, cudaStream_t st);


}  // namespace cxg
