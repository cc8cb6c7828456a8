"""A feed-forward made of experts: x += sum over the token's chosen experts of weight * W_down (silu(W_gate h) * (W_up h)).

The router's logits z = W_r h + b_r are computed in float32; the `top` experts with the largest logits are chosen (the
first of equal ones), and their weights are the softmax over the chosen logits only.  Experts have no biases.  The
step's (token, choice) pairs are grouped by expert on the device (no count ever reaches the host, so a step can be
replayed from a CUDA graph): each expert's rows start at a multiple of the products' row tile, the gate and up products
with the activation run over the grouped rows, the down product writes a float32 row per pair, and the weighted sum
into the residual stream takes a token's pairs in the order of its choices.
"""
import torch

from ..config.base import ConfigError
from ..csrc import ops
from . import linear
from .base import Part, as_matrix, as_vector, nbytes
from .registry import register_ffn


@register_ffn("moe")
class MixtureOfExperts(Part):
    graph_safe = True

    def __init__(self, spec, env):
        self.hidden, self.inter = spec["hidden_size"], spec["intermediate_size"]
        self.n_experts, self.top = spec["experts"], spec["top"]
        self.names = dict(spec["names"])
        self.dtype = env.dtype
        if self.n_experts < 1 or not 1 <= self.top <= self.n_experts or self.n_experts > 1024:
            raise ConfigError(f"moe: {self.top} of {self.n_experts} experts (up to 1024 experts)")
        self.w_gate = self.w_up = self.w_down = self.w_router = self.b_router = None

    def sizes(self):
        return {"intermediate": self.inter, "experts": self.n_experts, "experts_per_token": self.top}

    def flops(self, n_tokens, attended):
        return 2.0 * n_tokens * self.hidden * self.n_experts + 6.0 * n_tokens * self.top * self.hidden * self.inter

    def _expert(self, e, which):
        n = self.names
        return f"{n['expert']}{e}.{n[which]}"

    def weight_shapes(self, prefix):
        n, out = self.names, {}
        for e in range(self.n_experts):
            out[prefix + self._expert(e, "gate")] = (self.inter, self.hidden)
            out[prefix + self._expert(e, "up")] = (self.inter, self.hidden)
            out[prefix + self._expert(e, "down")] = (self.hidden, self.inter)
        out[prefix + n["router"]] = (self.n_experts, self.hidden)
        out[prefix + n["router_bias"]] = (self.n_experts,)
        return out

    def load(self, tensors, prefix, device):
        n = self.names
        stack = lambda which: torch.stack([as_matrix(tensors[prefix + self._expert(e, which)], self.dtype, device)
                                           for e in range(self.n_experts)]).contiguous()
        self.w_gate, self.w_up, self.w_down = stack("gate"), stack("up"), stack("down")
        self.w_router = as_matrix(tensors[prefix + n["router"]], torch.float32, device)
        self.b_router = as_vector(tensors[prefix + n["router_bias"]], device)

    def _on_tensor_cores(self):
        """Whether the experts' products run as grouped tcgen05 products (bfloat16 and sizes that kernel takes)."""
        return (self.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.inter % 8 == 0 and self.w_gate is not None and
                self.w_gate.data_ptr() % 16 == 0 and self.w_up.data_ptr() % 16 == 0 and self.w_down.data_ptr() % 16 == 0)

    def _max_tiles(self, n_tokens, tile_rows):
        return ops.moe_max_tiles(n_tokens * self.top, self.n_experts, tile_rows)

    def workspace_bytes(self, n_tokens, n_seqs):
        tile_rows = ops.moe_tile_rows(self._on_tensor_cores())
        tiles = self._max_tiles(n_tokens, tile_rows)
        rows, pairs = tiles * tile_rows, n_tokens * self.top
        return (nbytes((n_tokens, self.hidden), self.dtype) + 2 * nbytes((pairs,), torch.int32) + nbytes((pairs,), torch.float32) +
                nbytes((rows,), torch.int32) + nbytes((tiles,), torch.int32) + nbytes((rows, self.hidden), self.dtype) +
                nbytes((rows, self.inter), self.dtype) + nbytes((rows, self.hidden), torch.float32))

    def first_weights(self):
        return ()

    def forward(self, ctx, h, x, accumulate=True):
        h = linear.as_tensor(h)
        T, ws = h.shape[0], ctx.ws
        tc = self._on_tensor_cores()
        tile_rows = ops.moe_tile_rows(tc)
        max_tiles = self._max_tiles(T, tile_rows)
        rows = max_tiles * tile_rows
        idx = ws.alloc((T, self.top), torch.int32)
        wts = ws.alloc((T, self.top), torch.float32)
        row_pair = ws.alloc((rows,), torch.int32)
        pair_row = ws.alloc((T * self.top,), torch.int32)
        tile_expert = ws.alloc((max_tiles,), torch.int32)
        with ctx.prof("moe_route"):
            ops.moe_route(h, self.w_router, self.b_router, idx, wts, self.top)
            ops.moe_plan(idx, self.n_experts, tile_rows, row_pair, pair_row, tile_expert)
        mid = ws.alloc((rows, self.inter), self.dtype)
        y = ws.alloc((rows, self.hidden), torch.float32)
        if tc:
            a = ws.alloc((rows, self.hidden), self.dtype)
            with ctx.prof("moe_gather"):
                ops.moe_gather_rows(h, a, row_pair, self.top)
            with ctx.prof("moe_gate_up"):
                ops.gemm_tc_grouped(a, self.w_gate, mid, tile_expert, ctx.err, epilogue=linear.EPI_SWIGLU, w2=self.w_up)
            with ctx.prof("moe_down"):
                ops.gemm_tc_grouped(mid, self.w_down, y, tile_expert, ctx.err)
        else:
            with ctx.prof("moe_gate_up"):
                ops.moe_gate_up(h, self.w_gate, self.w_up, mid, row_pair, tile_expert, self.top)
            with ctx.prof("moe_down"):
                ops.moe_down(mid, self.w_down, y, row_pair, tile_expert, self.top)
        with ctx.prof("moe_combine"):
            if not accumulate:
                x.zero_()
            ops.moe_combine(x, y, wts, pair_row)
