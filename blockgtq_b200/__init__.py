"""blockgtq_b200: B200 (sm_100a) implementation of Block-GTQ's packed-KV-cache decode path
behind the reference's Python API.  All GPU work is done by ``libbgtq.so`` (hand-written CUDA,
C ABI in ``include/bgtq.h``); there is no CPU or Triton fallback."""
from .allocator import greedy_bit_allocation
from .quantizer import (BlockGTQQuantizer, build_batched_encode_args, build_pack_meta,
                        compress_k_mixed_batched, compress_k_packed_batched,
                        compress_v_nibble4_batched, compress_v_packed_batched)
from .attention import fused_blockgtq_decode_attention, fused_blockgtq_prefill_attention
from .packed_kv_manager import BlockGTQKVManager, decode_step
from .production_cache import BlockGTQProductionCache
from .production_decode import production_decode_step, production_prefill
from .prefill import layer_major_prefill
from .calibration import (bake_q_rotations, build_quantizers, collect_qk_activations, load_calib_cache,
                          save_calib_cache)

__all__ = [
    "greedy_bit_allocation", "BlockGTQQuantizer", "build_batched_encode_args", "build_pack_meta",
    "compress_k_packed_batched", "compress_v_packed_batched", "compress_k_mixed_batched",
    "compress_v_nibble4_batched", "fused_blockgtq_decode_attention", "BlockGTQKVManager", "decode_step",
    "BlockGTQProductionCache", "production_decode_step", "production_prefill", "collect_qk_activations",
    "build_quantizers", "bake_q_rotations", "fused_blockgtq_prefill_attention", "layer_major_prefill",
    "save_calib_cache", "load_calib_cache",
]
