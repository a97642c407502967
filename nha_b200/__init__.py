"""nha_b200: the NHA attention operator on hand-written CUDA kernels for B200 (sm_100a).

The public names and signatures are those of ``nha_fla.ops.nha`` so that the
reference's layers and model classes can call them unchanged.
"""
from .chunk import chunk_nha
from .chunk_fused import fused_chunk_nha_prefill
from .fused_recurrent import fused_recurrent_nha, fused_recurrent_nha_decode, fused_recurrent_nha_decode_bf16_state
from .gates import slot_gates
from .layer_ops import feature_maps, silu_rms_norm, silu_rms_norm_linear
from .lse_stats import gsa_aux_loss
from .rotary import rotary_pair
from .ring_cache import NHARingCache, fused_recurrent_nha_decode_ring
from .patch import WideWindow, patch_reference, route_wide_windows, unpatch_reference

__all__ = ['chunk_nha', 'fused_chunk_nha_prefill', 'fused_recurrent_nha', 'fused_recurrent_nha_decode',
           'fused_recurrent_nha_decode_ring', 'fused_recurrent_nha_decode_bf16_state', 'NHARingCache', 'slot_gates', 'rotary_pair', 'gsa_aux_loss',
           'feature_maps', 'silu_rms_norm', 'silu_rms_norm_linear', 'patch_reference', 'unpatch_reference', 'route_wide_windows', 'WideWindow']
__version__ = '0.1.0'
