"""B200-native Grouped Cross-Attention and landmark retrieval for the DRT model.

Host layer (this package) = views, strides, autograd bookkeeping; all arithmetic lives in
``libgca_b200.so`` (CUDA, sm_100a) behind the C ABI of ``include/gca_b200.h``.
"""
from .gca import (attention, gca_kv_cache, gca_indexed, gca_indexed_nograd, read_status, check_status,  # noqa: F401
                  set_status_checks)
from ._lib import GcaError, set_nvtx  # noqa: F401
from .retrieval import (lmk_score_topk, merge_topk, retrieve, perform_batch_retrieval,  # noqa: F401
                        decode_retrieval, differentiable_weights, Retrieval)
from .chunk_cache import ChunkKVManager  # noqa: F401
from .host_pipeline import HostGcaPipeline  # noqa: F401
from .modules import TritonGroupCrossAttention, GroupCrossAttention, preprocess_chunk_kv_cache  # noqa: F401
from . import fused_ops  # noqa: F401
