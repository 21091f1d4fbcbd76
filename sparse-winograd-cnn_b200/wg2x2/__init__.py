"""Host-side Python over libwinograd2x2_b200.so (B200 Winograd-ReLU F(2x2,3x3) convolution)."""
from . import _lib  # noqa: F401  (raises if the CUDA library is missing)
from ._lib import MATH_FP32, MATH_TF32, NCHW, NHWC, Wg2x2Error  # noqa: F401
from .ops import conv_bwd, conv_fwd, conv_fwd_prepared, prepare_weights, imtrans_bwd, imtrans_fwd, last_device_status, maxpool3x3s2_same, stem_prepare, stem7x7s2_pool, stem_supported, layer_fwd, layer_fwd_prepared, layer_fwd_prepared_workspace_bytes, layer_fwd_fused, fused_supported  # noqa: F401
from .host import HostLayerPipeline  # noqa: F401
from . import shard  # noqa: F401
