"""A gated linear recurrence (linear attention whose forget gate also decides what is written):
per head, with key size dk and value size dv,

    q_t = silu(Wq h_t),   f_t = l + (1 - l) sigmoid(Wf h_t + b),   v_t = Wv h_t,
    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,   o_t = S_t^T q_t,

l a lower bound per key channel (a stored tensor, as it is given), S [dk, dv] starting at zero.
Each head's o_t is normed over dv with one weight shared by the heads, the heads are
concatenated and projected by Wo.  The state is a fixed-size per-sequence cache need
(float32 [heads, dk, dv]); gates, state and the norm are 32-bit, the three projections are
one product over the stacked matrix [Wq; Wf; Wv].
"""
from __future__ import annotations

import torch

from ..cache import CacheNeed
from ..csrc import ops
from ..weights import TensorNeed
from .base import register_mixer
from .linear import matmul_partials


@register_mixer("gated_linear_recurrence")
class GatedLinearRecurrence:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.D = int(params["hidden_size"])
        self.H = int(params["num_heads"])
        self.dk = int(params["key_dim"])
        self.dv = int(params["value_dim"])
        self.eps = float(params["eps"])
        if min(self.H, self.dk, self.dv) <= 0 or self.dk > 512:
            raise ValueError(f"gated_linear_recurrence: heads {self.H}, key size {self.dk} (up to 512), "
                             f"value size {self.dv}")
        self.w_qfv = self.w_o = self.f_bias = self.lower = self.norm = None

    def tensor_needs(self):
        H, dk, dv, D = self.H, self.dk, self.dv, self.D
        return {"q": TensorNeed((H * dk, D)), "f": TensorNeed((H * dk, D)), "v": TensorNeed((H * dv, D)),
                "f.b": TensorNeed((H * dk,), init="around_zero"),
                "lower": TensorNeed((H * dk,), init="around_zero"),
                "norm": TensorNeed((dv,), init="ones"), "o": TensorNeed((D, H * dv))}

    def bind(self, tensors) -> None:
        parts = [tensors["q"], tensors["f"], tensors["v"]]
        if any(p.dtype == torch.float32 for p in parts):
            parts = [p.to(torch.float32) for p in parts]
        self.w_qfv = self.rt.matrix(torch.cat(parts, 0))
        self.w_o = self.rt.matrix(tensors["o"])
        self.f_bias = self.rt.vector(tensors["f.b"])
        self.lower = self.rt.vector(tensors["lower"])
        self.norm = self.rt.vector(tensors["norm"])

    def cache_need(self) -> CacheNeed:
        return CacheNeed("state", state_shape=(self.H, self.dk, self.dv), state_dtype=torch.float32)

    def cache_read_bytes(self, contexts, element_size: int) -> int:
        return 2 * len(contexts) * self.H * self.dk * self.dv * 4        # the state, read and written

    def flops(self, q_lens, past) -> float:
        n = sum(q_lens)
        return 2.0 * n * ((2 * self.dk + self.dv) * self.H * self.D + self.D * self.H * self.dv) \
            + 4.0 * n * self.H * self.dk * self.dv

    def forward(self, h, batch, stream, view, shared: bool = False):
        if shared:
            raise RuntimeError("a recurrent state cannot be read by another run entry")
        rt, H, dk, dv = self.rt, self.H, self.dk, self.dv
        n = batch.n_tokens
        proj, S = matmul_partials(rt, h, self.w_qfv, "recurrence_qfv")
        o = rt.buffer("recurrence_out", (n, H * dv), torch.float32)
        act = rt.buffer("recurrence_act", (n, 2 * H * dk + H * dv), torch.float32)
        ops.gated_recurrence(proj, S, self.f_bias, self.lower, batch, view.state, o, H, dk, dv, act)
        on = rt.buffer("recurrence_normed", (n, H * dv), rt.dtype)
        ops.head_norm(o, self.norm, on, H, dv, self.eps)
        stream.add_linear(on, self.w_o)
        return None
