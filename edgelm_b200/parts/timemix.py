"""Time mixing with a matrix-valued state and a decay that depends on the token (in the manner of RWKV).

With h' the previous token's input (zeros before a sequence's first token), each of r, k, v, g, w reads its own
blend h + (h' - h) * mu_s.  r, k, v are projections of their blends, heads x head_dim each; gate = silu(W_g blend_g);
the decay is w = exp(-exp(W_w2 tanh(W_w1 blend_w) + w0)), per head and key channel.  Per head, with bonus u:

    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t          (the bonus counts for the current token only)
    S_t = diag(w_t) S_(t-1) + k_t v_t^T                (S is head_dim x head_dim, float32, zero at the start)

Each head's o is divided by its root mean square; the heads, side by side, times a weight, times the gate, are
projected back.  A sequence's state: S per head and the last token's input h.  Decays, the recurrence and the norm are
float32 in both precisions; r, k, v, the gate and the decay's first projection are matrix products in the compute
dtype whose float32 sums are kept; the decay's second (low-rank) product runs in float32 on the CUDA cores.
"""
import torch

from ..config.base import ConfigError
from ..csrc import ops
from . import linear
from .base import NeedSet, Part, StateNeed, as_matrix, as_vector, nbytes
from .registry import register_mixer

BLENDS = ("r", "k", "v", "g", "w")


@register_mixer("decay_timemix")
class DecayTimeMix(Part):
    graph_safe = True

    def __init__(self, spec, env):
        self.hidden, self.heads, self.head_dim, self.rank = spec["hidden_size"], spec["heads"], spec["head_dim"], spec["decay_rank"]
        self.eps = float(spec["eps"])
        self.names = dict(spec["names"])
        self.dtype = env.dtype
        if self.heads < 1 or not 1 <= self.head_dim <= 256 or self.rank < 1:
            raise ConfigError(f"decay_timemix: {self.heads} heads of {self.head_dim} with a decay rank of {self.rank} are not taken (head size up to 256)")
        self.inner = self.heads * self.head_dim

    def sizes(self):
        return {"timemix_heads": self.heads, "timemix_head_dim": self.head_dim, "decay_rank": self.rank}

    def flops(self, n_tokens, attended):
        proj = 2.0 * n_tokens * self.hidden * (5 * self.inner + self.rank) + 2.0 * n_tokens * self.rank * self.inner
        return proj + 6.0 * n_tokens * self.inner * self.head_dim

    def weight_shapes(self, prefix):
        n, out = self.names, {}
        for s in BLENDS:
            out[prefix + n["mu"] + s] = (self.hidden,)
        for s in ("r", "k", "v", "g"):
            out[prefix + n[s]] = (self.inner, self.hidden)
        out[prefix + n["w1"]] = (self.rank, self.hidden)
        out[prefix + n["w2"]] = (self.inner, self.rank)
        out[prefix + n["w0"]] = (self.inner,)
        out[prefix + n["bonus"]] = (self.heads, self.head_dim)
        out[prefix + n["norm"]] = (self.inner,)
        out[prefix + n["out"]] = (self.hidden, self.inner)
        return out

    def load(self, tensors, prefix, device):
        n = self.names
        self.mu = torch.stack([as_vector(tensors[prefix + n["mu"] + s], device) for s in BLENDS]).contiguous()
        self.w = {s: as_matrix(tensors[prefix + n[s]], self.dtype, device) for s in ("r", "k", "v", "g", "w1", "w2", "out")}
        self.w0 = as_vector(tensors[prefix + n["w0"]], device)
        self.bonus = as_matrix(tensors[prefix + n["bonus"]], torch.float32, device)
        self.norm_w = as_vector(tensors[prefix + n["norm"]], device)

    def first_weights(self):
        return (self.w["r"],)

    def cache_need(self):
        return NeedSet.of(last=StateNeed((self.hidden,)), wkv=StateNeed((self.heads, self.head_dim, self.head_dim)))

    def workspace_bytes(self, n_tokens, n_seqs):
        f32 = torch.float32
        return (nbytes((5, n_tokens, self.hidden), self.dtype) + 6 * nbytes((n_tokens, self.inner), f32) + nbytes((n_tokens, self.rank), f32) +
                nbytes((n_tokens, self.inner), self.dtype) + nbytes((n_tokens, self.hidden), self.dtype))

    def forward(self, ctx, h, x, cache, accumulate=True):
        h = linear.as_tensor(h)
        T, ws, f32 = h.shape[0], ctx.ws, torch.float32
        blends = ws.alloc((5, T, self.hidden), self.dtype)
        last = cache["last"].state
        with ctx.prof("timemix_blend"):
            ops.shift_mix(h, last, self.mu, blends, ctx.tok_seq, ctx.seq_tok0, ctx.seq_slots, move_state=True)
        proj = {}
        with ctx.prof("timemix_proj"):
            for i, s in enumerate(("r", "k", "v", "g")):
                proj[s] = ws.alloc((T, self.inner), f32)
                linear.matmul(ctx, blends[i], self.w[s], proj[s])
            low = ws.alloc((T, self.rank), f32)
            linear.matmul(ctx, blends[4], self.w["w1"], low)
        decay = ws.alloc((T, self.inner), f32)
        with ctx.prof("timemix_decay"):
            ops.lowrank_decay(low, self.w["w2"], self.w0, decay)
        o = ws.alloc((T, self.inner), f32)
        with ctx.prof("timemix_scan"):
            ops.wkv_scan(proj["r"], proj["k"], proj["v"], decay, self.bonus, cache["wkv"].state, o, ctx.seq_tok0, ctx.seq_slots, ctx.n_seqs,
                         self.heads, self.head_dim)
        on = ws.alloc((T, self.inner), self.dtype)
        with ctx.prof("timemix_gate_norm"):
            ops.gated_group_norm(o, proj["g"], self.norm_w, on, self.heads, self.eps, gate_first=False)
        with ctx.prof("timemix_out_proj"):
            linear.matmul(ctx, on, self.w["out"], x, epilogue=linear.EPI_RESIDUAL if accumulate else linear.EPI_STORE,
                          residual=x if accumulate else None, prefetch=ctx.weights_after)
