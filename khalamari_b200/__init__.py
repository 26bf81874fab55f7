"""khalamari_b200: paged GQA split-KV scaled-dot-product attention for NVIDIA B200.

The product is ``libkhcuda_gqa.so`` (CUDA kernels for sm_100a behind the C ABI of ``include/kh_gqa.h``).
The modules here mirror, over that ABI, the reference interfaces the path is reached through:

==========================  =====================================================================
module                      reference file
==========================  =====================================================================
``sdpa``                    crates/inference-backend-metal/src/components/gqa/sdpa.rs
``sliced_kv``               crates/inference-backend-metal/src/components/gqa/sdpa/sliced_kv.rs
``sliced_q``                crates/inference-backend-metal/src/components/gqa/sdpa/sliced_q.rs
``selector``                crates/inference-executor-metal/src/attn/gqa/sdpa.rs
``batch_metadata``          crates/inference-executor-metal/src/attn/gqa/batch_metadata.rs
``request_page_table``      crates/inference-executor-metal/src/attn/gqa/request_page_table.rs
``replay``                  crates/inference-executor-core/src/replay.rs
``gqa``                     crates/inference-executor-metal/src/attn/gqa/backend.rs (prepare, record_sdpa)
``device``                  crates/inference-backend-metal/src/metal/{device,buffer,stream}
==========================  =====================================================================
"""
from . import abi  # noqa: F401

__all__ = ["abi"]
