"""mononn_b200: B200 (sm_100a) backend for the MonoNN hot path -- an XLA HLO module in,
one persistent kernel launch per inference out.  The work is done by libmononn_b200.so
(mononn_b200/csrc); this package is the thin host-side mirror of its C ABI."""
from .capi import MononnError, Options  # noqa: F401
from .module import Module, compile_encoder, compile_hlo  # noqa: F401
from .models import (ClipConfig, EncoderConfig, bert_base, bert_tiny, clip_b32, clip_tiny,  # noqa: F401
                     make_clip_inputs, make_inputs, make_vit_inputs, make_weights, opt_1p3b, opt_tiny,
                     make_t5_inputs, t5_device_weights, t5_small, t5_tiny, vit_base, vit_tiny)
