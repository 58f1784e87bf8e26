"""NN library (zml/nn.zig of the reference): linear + quantisation schemes, norms,
activations, RoPE, sdpa, GatedDeltaNet, sampling, image resizing."""
from .attention_ref import GatedDeltaNetOutput, causal_attn_mask, gated_delta_net, sdpa  # noqa: F401
from .image import nearest, resize_bicubic, resize_bilinear, upsample  # noqa: F401
from .layers import (Activation, LayerNorm, Linear, Quant, TensorScale, TokenEmbedding, normalize_l2,  # noqa: F401
                     normalize_variance, rms_norm)
from .quant import (NVFP4_BLOCK, QuantScheme, dequantize_nvfp4, is_packed_nvfp4, quantize_nvfp4,  # noqa: F401
                    quantize_weight_nvfp4, scaled_dot)
from .rotary import (Layout, RopeOpts, Scaling, inv_freq, merge_real_img, merge_real_img_pass, rope,  # noqa: F401
                     split_real_img, split_real_img_pass)
from .sampling import (DynamicSamplingStrategy, SamplingStrategy, fixup_logits, sample_tokens,  # noqa: F401
                       sample_tokens_dynamic)
