"""NN library (zml/nn.zig of the reference): linear + quantisation schemes, norms,
activations, RoPE, sdpa, GatedDeltaNet, sampling, image resizing."""
from .rotary import Layout, RopeOpts, Scaling, inv_freq, rope  # noqa: F401
