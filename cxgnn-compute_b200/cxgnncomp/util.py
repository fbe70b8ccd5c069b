import logging

from .codegen import Tuner

log = logging.getLogger(__name__)
global_tuner = Tuner(lazy=True)
