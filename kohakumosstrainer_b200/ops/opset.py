"""The op-set interface and its eager implementation.

A block calls layer-level ops that take the `MossLinear` modules themselves
(`qkv_rope`, `linear_situ`, `linear_gated_residual`), so an implementation is free to fuse
the GEMM with its epilogue, the adapter bypass and the activation quantiser. The eager
op set composes the primitives exactly as the reference does
(`src/kohakumoss/model/opset.py:94-124`).
"""

from __future__ import annotations

from torch import Tensor

from . import eager


class OpSet:
    name = "abstract"

    # primitives
    rms_norm = staticmethod(eager.rms_norm)
    rms_norm_mod = staticmethod(eager.rms_norm_mod)
    qk_norm_rope = staticmethod(eager.qk_norm_rope)
    situ_glu = staticmethod(eager.situ_glu)
    situ_pair = staticmethod(eager.situ_pair)
    gated_residual = staticmethod(eager.gated_residual)
    token_mse = staticmethod(eager.token_mse)
    attention_varlen = staticmethod(eager.attention_varlen)

    def attention(self, q: Tensor, k: Tensor, v: Tensor, plan) -> Tensor:
        """Packed attention over the segments of `plan`, softmax scale Dh^-0.5."""
        return self.attention_varlen(
            q, k, v, plan.cu_seqlens, plan.max_seqlen, q.shape[-1] ** -0.5, plan.lengths
        )

    # layer-level ops
    def qkv_rope(self, y, lin_q, lin_k, lin_v, heads, q_weight, k_weight, pos, bands, eps):
        q = lin_q(y).unflatten(-1, (heads, -1))
        k = lin_k(y).unflatten(-1, (heads, -1))
        v = lin_v(y).unflatten(-1, (heads, -1))
        q, k = self.qk_norm_rope(q, k, q_weight, k_weight, pos, bands, eps)
        return q, k, v

    def linear_situ(self, y, lin):
        return self.situ_glu(lin(y))

    def linear_gated_residual(self, a, lin, x, gate, seg, r):
        return self.gated_residual(x, lin(a), gate, seg, r)


class EagerOps(OpSet):
    name = "eager"
