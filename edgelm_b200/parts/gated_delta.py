"""The gated delta rule: a recurrent mixer with a matrix-valued state that is corrected, not only added to.

q = W_q h and k = W_k h (`kv_heads` heads of `head_dim`), v = W_v h (`heads` heads of `v_head_dim`); value head n uses
query/key head n // (heads / kv_heads).  Each of q, k, v passes a short causal convolution per channel (taps from a
[channels, taps] tensor whose last column multiplies the current token, no bias, zeros before a sequence's start) and
silu.  Then q and k become unit vectors per head, x / sqrt(sum(x^2) + unit_eps), and q is multiplied by head_dim^(-1/2).
Per value head, with beta = sigmoid(W_b h) and the decay g = exp(-exp(A_log) softplus(W_a h + dt_bias)):

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q           (S is head_dim x v_head_dim, zero at the start)

so the read-out sees the token's own write.  Each head's o is divided by its root mean square (eps), times a weight of
size v_head_dim that the heads share, times silu(W_g h); then the output projection.  A sequence's state: S per head and
the convolutions' last taps - 1 inputs.  Decays, step sizes, unit norms, the recurrence and the norm are float32 in both
precisions; the projections run in the compute dtype and their float32 sums are kept.
"""
import torch

from ..config.base import ConfigError
from ..csrc import ops
from . import linear
from .base import NeedSet, Part, StateNeed, as_matrix, as_vector, nbytes
from .registry import register_mixer

UNIT_EPS = 1e-6     # inside the root of the unit norm of queries and keys


@register_mixer("gated_delta")
class GatedDelta(Part):
    graph_safe = True

    def __init__(self, spec, env):
        self.hidden = spec["hidden_size"]
        self.heads, self.kv_heads, self.d, self.e, self.taps = spec["heads"], spec["kv_heads"], spec["head_dim"], spec["v_head_dim"], spec["conv"]
        self.eps, self.unit_eps = float(spec["eps"]), float(spec.get("unit_eps", UNIT_EPS))
        self.names = dict(spec["names"])
        self.dtype = env.dtype
        if self.heads < 1 or self.kv_heads < 1 or self.heads % self.kv_heads:
            raise ConfigError(f"gated_delta: {self.heads} value heads are not a multiple of {self.kv_heads} query/key heads")
        if not 1 <= self.d <= 256 or self.e < 1 or self.taps < 1:
            raise ConfigError(f"gated_delta: heads of {self.d} x {self.e} with {self.taps} taps are not taken (key size up to 256)")
        self.qk, self.inner = self.kv_heads * self.d, self.heads * self.e
        self.channels = 2 * self.qk + self.inner              # what the convolutions see: q | k | v
        self.b_off, self.a_off, self.g_off = self.channels, self.channels + self.heads, self.channels + 2 * self.heads
        self.d_in = self.channels + 2 * self.heads + self.inner     # q | k | v | b | a | gate

    def sizes(self):
        return {"delta_heads": self.heads, "delta_kv_heads": self.kv_heads, "delta_head_dim": self.d, "delta_v_head_dim": self.e,
                "conv_taps": self.taps}

    def flops(self, n_tokens, attended):
        return 2.0 * n_tokens * self.hidden * (self.d_in + self.inner) + 6.0 * n_tokens * self.inner * self.d

    def weight_shapes(self, prefix):
        n = self.names
        return {prefix + n["q"]: (self.qk, self.hidden), prefix + n["k"]: (self.qk, self.hidden), prefix + n["v"]: (self.inner, self.hidden),
                prefix + n["q"] + n["conv"]: (self.qk, self.taps), prefix + n["k"] + n["conv"]: (self.qk, self.taps),
                prefix + n["v"] + n["conv"]: (self.inner, self.taps), prefix + n["b"]: (self.heads, self.hidden),
                prefix + n["a"]: (self.heads, self.hidden), prefix + n["A_log"]: (self.heads,), prefix + n["dt_bias"]: (self.heads,),
                prefix + n["g"]: (self.inner, self.hidden), prefix + n["norm"]: (self.e,), prefix + n["o"]: (self.hidden, self.inner)}

    def load(self, tensors, prefix, device):
        n = self.names
        # every projection of the mixer's input in one product: q | k | v | b | a | gate
        self.w_in = torch.cat([as_matrix(tensors[prefix + n[k]], self.dtype, device) for k in ("q", "k", "v", "b", "a", "g")], dim=0).contiguous()
        self.conv_w = torch.cat([as_matrix(tensors[prefix + n[k] + n["conv"]], torch.float32, device) for k in ("q", "k", "v")], dim=0).contiguous()
        self.conv_b = torch.zeros(self.channels, dtype=torch.float32, device=device)
        self.no_tail = torch.zeros((1, 0, self.channels), dtype=torch.float32, device=device)   # (one tap: no earlier input is kept)
        self.a_log = as_vector(tensors[prefix + n["A_log"]], device)
        self.dt_bias = as_vector(tensors[prefix + n["dt_bias"]], device)
        self.norm_w = as_vector(tensors[prefix + n["norm"]], device).repeat(self.heads).contiguous()   # the heads share it
        self.w_o = as_matrix(tensors[prefix + n["o"]], self.dtype, device)

    def first_weights(self):
        return (self.w_in,)

    def cache_need(self):
        return NeedSet.of(conv=StateNeed((self.taps - 1, self.channels)) if self.taps > 1 else None,
                          delta=StateNeed((self.heads, self.e, self.d)))

    def workspace_bytes(self, n_tokens, n_seqs):
        f32 = torch.float32
        return (nbytes((n_tokens, self.d_in), f32) + nbytes((n_tokens, self.channels), f32) + nbytes((n_tokens, self.inner), f32) +
                nbytes((2 * n_tokens * self.heads,), f32) + nbytes((n_tokens, self.inner), self.dtype) + nbytes((n_tokens, self.hidden), self.dtype))

    def forward(self, ctx, h, x, cache, accumulate=True):
        h = linear.as_tensor(h)
        T, ws, f32 = h.shape[0], ctx.ws, torch.float32
        u = ws.alloc((T, self.d_in), f32)
        with ctx.prof("delta_in_proj"):
            linear.matmul(ctx, h, self.w_in, u, prefetch=(self.w_o,))
        qkv = ws.alloc((T, self.channels), f32)
        conv = cache.get("conv")
        with ctx.prof("delta_conv"):
            ops.conv_silu(u, 0, self.conv_w, self.conv_b, conv.state if conv is not None else self.no_tail, qkv,
                          ctx.tok_seq, ctx.seq_tok0, ctx.seq_slots, ctx.n_seqs, update_state=True)
        bg = ws.alloc((2 * T * self.heads,), f32)
        with ctx.prof("delta_prepare"):
            ops.delta_prepare(qkv, u, self.b_off, self.a_off, self.a_log, self.dt_bias, bg, self.heads, self.kv_heads, self.d, self.e,
                              self.unit_eps, float(self.d) ** -0.5)
        o = ws.alloc((T, self.inner), f32)
        with ctx.prof("delta_scan"):
            ops.delta_scan(qkv, bg, cache["delta"].state, o, ctx.seq_tok0, ctx.seq_slots, ctx.n_seqs, self.heads, self.kv_heads, self.d, self.e)
        on = ws.alloc((T, self.inner), self.dtype)
        with ctx.prof("delta_gate_norm"):
            ops.gated_group_norm(o, u[:, self.g_off:], self.norm_w, on, self.heads, self.eps, gate_first=False)
        with ctx.prof("delta_out_proj"):
            linear.matmul(ctx, on, self.w_o, x, epilogue=linear.EPI_RESIDUAL if accumulate else linear.EPI_STORE,
                          residual=x if accumulate else None, prefetch=ctx.weights_after)
