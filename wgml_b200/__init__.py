"""wgml_b200: the per-token transformer forward of wgml as hand-written sm_100a CUDA kernels behind
a C ABI (include/wgml_b200.h), with a host-side mirror of wgml's operator structs.

`wgml_b200.ops`     GemvQuant, RmsNorm, LayerNorm, RoPE, BatchedMultiqueryAttention, SoftMax, Silu, Unary, OpAssign
`wgml_b200.models`  Llama2 / Gpt2 decoders and their configs
`wgml_b200.gguf`    GGUF reader
`wgml_b200.synth`   seeded synthetic weights for the benchmark configurations
"""
from ._lib import WgbError, load  # noqa: F401

__all__ = ["WgbError", "load"]
