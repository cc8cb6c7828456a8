"""Selective state-space mixer in the state-space-duality form (Mamba-2).

With inner = heads * head_dim, N the state size and G the groups, one input projection gives, side by side,
[z: inner | x: inner | B: G N | C: G N | dt: heads].  x, B and C pass a causal convolution per channel (taps from a
[channels, taps] tensor whose last column multiplies the current token, a bias, zeros before a sequence's start)
and silu.  Per head h (group h // (heads / G)), with dt = softplus(dt + dt_bias_h), without a clamp:

    S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T          (S is N x head_dim, float32, zero at the start)
    y_t = S_t^T C_t + D_h x_t

The heads' y, side by side, are multiplied by silu(z), THEN divided by their root mean square in `norm_groups` equal
parts, times a weight, and projected back.  A sequence's state: S per head, and the convolution's last taps - 1
inputs.  The step sizes, decays, the recurrence and the norm are float32 in both precisions; the two projections run
in the compute dtype with float32 sums, and the input projection's result stays float32.
"""
import torch

from ..config.base import ConfigError
from ..csrc import ops
from . import linear
from .base import NeedSet, Part, StateNeed, as_matrix, as_vector, nbytes
from .registry import register_mixer


@register_mixer("mamba2")
class Mamba2(Part):
    graph_safe = True

    def __init__(self, spec, env):
        self.hidden = spec["hidden_size"]
        self.heads, self.head_dim, self.n_state = spec["heads"], spec["head_dim"], spec["state"]
        self.groups, self.taps, self.norm_groups = spec["groups"], spec["conv"], spec["norm_groups"]
        self.eps = float(spec["eps"])
        self.names = dict(spec["names"])
        self.dtype = env.dtype
        for name in ("heads", "head_dim", "n_state", "groups", "taps", "norm_groups"):
            if getattr(self, name) < 1:
                raise ConfigError(f"mamba2: {name} must be positive, found {getattr(self, name)}")
        if self.heads % self.groups:
            raise ConfigError(f"mamba2: {self.heads} heads are not a multiple of {self.groups} groups")
        self.inner = self.heads * self.head_dim
        if self.inner % self.norm_groups:
            raise ConfigError(f"mamba2: {self.inner} inner channels do not split into {self.norm_groups} equal norm groups")
        if self.n_state > 256:
            raise ConfigError(f"mamba2: a state of {self.n_state} rows per head is not taken by the scan kernel (up to 256)")
        self.channels = self.inner + 2 * self.groups * self.n_state      # what the convolution sees: x | B | C
        self.d_in = 2 * self.inner + 2 * self.groups * self.n_state + self.heads
        self.w_in = self.w_o = None

    def sizes(self):
        return {"ssm_heads": self.heads, "ssm_head_dim": self.head_dim, "ssm_state": self.n_state, "ssm_groups": self.groups,
                "conv_taps": self.taps, "norm_groups": self.norm_groups}

    def flops(self, n_tokens, attended):
        proj = 2.0 * n_tokens * self.hidden * (self.d_in + self.inner)
        scan = 6.0 * n_tokens * self.inner * self.n_state
        return proj + scan

    def weight_shapes(self, prefix):
        n = self.names
        return {prefix + n["in"]: (self.d_in, self.hidden), prefix + n["conv"]: (self.channels, self.taps),
                prefix + n["conv_bias"]: (self.channels,), prefix + n["dt_bias"]: (self.heads,), prefix + n["A_log"]: (self.heads,),
                prefix + n["D"]: (self.heads,), prefix + n["norm"]: (self.inner,), prefix + n["out"]: (self.hidden, self.inner)}

    def load(self, tensors, prefix, device):
        n = self.names
        self.w_in = as_matrix(tensors[prefix + n["in"]], self.dtype, device)
        self.w_o = as_matrix(tensors[prefix + n["out"]], self.dtype, device)
        self.conv_w = as_matrix(tensors[prefix + n["conv"]], torch.float32, device)
        self.conv_b = as_vector(tensors[prefix + n["conv_bias"]], device)
        self.dt_bias = as_vector(tensors[prefix + n["dt_bias"]], device)
        self.a_log = as_vector(tensors[prefix + n["A_log"]], device)
        self.d = as_vector(tensors[prefix + n["D"]], device)
        self.norm_w = as_vector(tensors[prefix + n["norm"]], device)

    def first_weights(self):
        return (self.w_in,)

    def cache_need(self):
        return NeedSet.of(conv=StateNeed((self.taps - 1, self.channels)), ssm=StateNeed((self.heads, self.head_dim, self.n_state)))

    def workspace_bytes(self, n_tokens, n_seqs):
        f32 = torch.float32
        return (nbytes((n_tokens, self.d_in), f32) + nbytes((n_tokens, self.channels), f32) + nbytes((n_tokens, self.inner), f32) +
                nbytes((2 * n_tokens * self.heads,), f32) +
                nbytes((n_tokens, self.inner), self.dtype) + nbytes((n_tokens, self.hidden), self.dtype))

    def forward(self, ctx, h, x, cache, accumulate=True):
        h = linear.as_tensor(h)
        T, ws, f32 = h.shape[0], ctx.ws, torch.float32
        u = ws.alloc((T, self.d_in), f32)
        with ctx.prof("ssm_in_proj"):
            linear.matmul(ctx, h, self.w_in, u, prefetch=(self.w_o,))
        xbc = ws.alloc((T, self.channels), f32)
        with ctx.prof("ssm_conv"):
            ops.conv_silu(u, self.inner, self.conv_w, self.conv_b, cache["conv"].state, xbc, ctx.tok_seq, ctx.seq_tok0, ctx.seq_slots, ctx.n_seqs,
                          update_state=False)     # (the scan kernel moves the tail on)
        y = ws.alloc((T, self.inner), f32)
        steps = ws.alloc((2 * T * self.heads,), f32)
        with ctx.prof("ssm_scan"):
            ops.ssm_scan(xbc, u, 2 * self.inner + 2 * self.groups * self.n_state, self.dt_bias, self.a_log, self.d, cache["ssm"].state, y,
                         ctx.seq_tok0, ctx.seq_slots, ctx.n_seqs, self.heads, self.groups, self.n_state, self.head_dim,
                         conv_state=cache["conv"].state, conv_off=self.inner, scratch=steps)
        yn = ws.alloc((T, self.inner), self.dtype)
        with ctx.prof("ssm_gate_norm"):
            ops.gated_group_norm(y, u[:, :self.inner], self.norm_w, yn, self.norm_groups, self.eps, gate_first=True)
        with ctx.prof("ssm_out_proj"):
            linear.matmul(ctx, yn, self.w_o, x, epilogue=linear.EPI_RESIDUAL if accumulate else linear.EPI_STORE,
                          residual=x if accumulate else None, prefetch=ctx.weights_after)
