"""B200-native dense forward attention (bf16, head_dim 128) behind the reference's surfaces.

    ops.attention(q, k, v, ...)            tensors -> C ABI (ctypes), any strided layout
    registry.load_kernel()                 `module.sdpa(Q, K, V)` like the reference registry
    backend.B200Attention()                the video model's attention callable
    sharding / ring                        (batch, head) sharding and the K/V ring across GPUs

Importing the package loads nothing native; the first call does, and fails loudly if the
libraries have not been built (`python -m b200_attention_b200.build`).
"""

__version__ = "0.1.0"
