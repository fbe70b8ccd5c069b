import cxgnncomp_backend


def typed_matmul(a, b, rel, num_valid_item=-1, src_idx=None, dst_idx=None, seq_output=False):
    """C[out(m)] = A[in(m)] @ b[rel of m's 128-block], same arguments as the reference's typed_matmul
    (cxgnncomp/codegen/triton_typed_matmul.py:752-860):
      src_idx None                      in(m) = out(m) = m
      src_idx, dst_idx None             in(m) = src_idx[m]; out(m) = src_idx[m], or m with seq_output
      src_idx and dst_idx               in(m) = src_idx[m]; out(m) = dst_idx[m]
    `rel` holds the relation of every position, sorted so that aligned blocks of 128 positions share one
    relation; positions whose index is negative or >= num_valid_item are padding. Unlike the reference,
    which launches cdiv(num_valid_item, BLOCK_M) tiles over the padded array and so skips the last
    positions (its FIXME at :777), every position of `rel` is visited.
    bf16 inputs are multiplied as bf16 on the tensor cores; fp32 inputs as error-compensated TF32 (fp32 accuracy),
    or as plain TF32 like the reference's tl.dot when cxgnncomp_backend.ALLOW_TF32 is set."""
    assert a.shape[1] == b.shape[1], "incompatible dimensions"
    assert a.is_contiguous() and b.is_contiguous() and rel.is_contiguous()
    positions = rel.shape[0]
    if src_idx is not None:
        positions = min(positions, src_idx.shape[0])
    m_valid = num_valid_item if num_valid_item != -1 else (src_idx.shape[0] if src_idx is not None else a.shape[0])
    return cxgnncomp_backend.typed_matmul_raw(a, b, rel, positions, m_valid, src_idx=src_idx, dst_idx=dst_idx,
                                              seq_output=seq_output)
