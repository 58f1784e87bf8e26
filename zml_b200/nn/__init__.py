"""NN library (zml/nn.zig of the reference): linear + quantisation schemes, norms,
activations, RoPE, sdpa, GatedDeltaNet, sampling, image resizing."""
from .attention_ref import GatedDeltaNetOutput, causal_attn_mask, gated_delta_net, sdpa  # noqa: F401
from .image import (nearest, resize_bicubic, resize_bilinear, resize_cubic_1d, resize_linear_1d,  # noqa: F401
                    upsample)
from .layers import (DIM_MISMATCH, NOT_SET, Activation, LayerNorm, Linear, Quant, TensorScale,  # noqa: F401
                     TokenEmbedding, collect_dims, elu, normalize_l2, normalize_variance, rms_norm)
from .quant import (NVFP4_BLOCK, QuantScheme, dequantize_nvfp4, is_packed_nvfp4, quantize_nvfp4,  # noqa: F401
                    quantize_weight_nvfp4, scaled_dot, unpack_nvfp4)
from .rotary import (Layout, RopeOpts, Scaling, inv_freq, merge_real_img, merge_real_img_pass, rope,  # noqa: F401
                     split_real_img, split_real_img_pass)
from .sampling import (DynamicSamplingStrategy, SamplingStrategy, fixup_logits, sample_tokens,  # noqa: F401
                       sample_tokens_dynamic)
