"""Grouped-query attention over a sliding window with pooled blocks behind it.

q, k, v are projections with optional biases (one matrix product over the three weights stacked; its float32 sums are
kept, and the bias is added to them).  The first `rot_dims` dimensions of every query and key head are rotated by
position * f_i, f_i = base^(-2i / rot_dims) / scaling, dimension i paired with i + rot_dims/2; after that each query and
key head is divided by its root mean square (`unit_norm`).  Position i sees the keys j with 0 <= i - j < window and, for
every block of `pool` positions that lies wholly before the window, one key and value: the mean of the block's keys
(values) as the cache holds them.  Tokens that left the window and whose block is not yet seen are not seen at all.
One softmax over tokens and blocks, score = (q . k) * scale.  Angles, norms, scores and the softmax are float32.

The cache keeps every key and value in pages (a value head may have another size than a key head) and the pooled rows
beside them; a block's row is written in the step that brings the block's last position.
"""
import torch

from ..config.base import ConfigError
from ..csrc import ops
from . import linear
from .base import KVNeed, Part, as_matrix, as_vector, nbytes
from .registry import register_mixer


@register_mixer("pooled_window_attention")
class PooledWindowAttention(Part):
    graph_safe = True

    def __init__(self, spec, env):
        self.hidden = spec["hidden_size"]
        self.nh, self.nkv, self.dk, self.dv = spec["num_heads"], spec["num_kv_heads"], spec["head_dim"], spec["v_head_dim"]
        self.window, self.pool = int(spec["window"]), spec.get("pool")
        self.pool = int(self.pool) if self.pool else None
        self.scale = float(spec["scale"])
        self.rot, self.base, self.scaling = int(spec.get("rot_dims") or 0), float(spec.get("rot_base") or 10000.0), float(spec.get("rot_scaling") or 1.0)
        self.unit_norm, self.eps = bool(spec.get("unit_norm", False)), float(spec.get("eps") or 0.0)
        self.bias = bool(spec.get("bias", False))
        self.names = dict(spec["names"])
        self.dtype = env.dtype
        if self.nh <= 0 or self.nkv <= 0 or self.nh % self.nkv:
            raise ConfigError(f"pooled_window_attention: {self.nh} query heads are not a multiple of {self.nkv} key/value heads")
        if not (1 <= self.dk <= 256 and 1 <= self.dv <= 256):
            raise ConfigError(f"pooled_window_attention: head sizes {self.dk} / {self.dv} are not taken (1 to 256)")
        if self.rot % 2 or not 0 <= self.rot <= self.dk:
            raise ConfigError(f"pooled_window_attention: {self.rot} rotated dimensions of a head of {self.dk}")
        if self.window < 1 or (self.pool is not None and self.pool < 1):
            raise ConfigError(f"pooled_window_attention: a window of {self.window} keys, blocks of {self.pool}")
        self.d_qkv = (self.nh + self.nkv) * self.dk + self.nkv * self.dv
        self.freq = self.b_qkv = None
        self.tile_tokens = max(1, 32 // (self.nh // self.nkv))   # tokens whose heads fill one block of the prompt kernel

    def tile_sizes(self):
        return (self.tile_tokens,)

    def sizes(self):
        return {"heads": self.nh, "kv_heads": self.nkv, "head_dim": self.dk, "v_head_dim": self.dv, "window": self.window,
                "pool": self.pool or 0, "rot_dims": self.rot}

    def flops(self, n_tokens, attended):
        proj = 2.0 * n_tokens * self.hidden * (self.d_qkv + self.nh * self.dv)
        seen = min(attended, n_tokens * self.window) + (attended / self.pool if self.pool else 0)
        return proj + 2.0 * seen * self.nh * (self.dk + self.dv)

    def weight_shapes(self, prefix):
        n = self.names
        out = {prefix + n["q"]: (self.nh * self.dk, self.hidden), prefix + n["k"]: (self.nkv * self.dk, self.hidden),
               prefix + n["v"]: (self.nkv * self.dv, self.hidden), prefix + n["o"]: (self.hidden, self.nh * self.dv)}
        if self.bias:
            out.update({prefix + n["q"] + n["bias"]: (self.nh * self.dk,), prefix + n["k"] + n["bias"]: (self.nkv * self.dk,),
                        prefix + n["v"] + n["bias"]: (self.nkv * self.dv,)})
        return out

    def load(self, tensors, prefix, device):
        n = self.names
        self.w_qkv = torch.cat([as_matrix(tensors[prefix + n[k]], self.dtype, device) for k in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = as_matrix(tensors[prefix + n["o"]], self.dtype, device)
        if self.bias:
            self.b_qkv = torch.cat([as_vector(tensors[prefix + n[k] + n["bias"]], device) for k in ("q", "k", "v")]).contiguous()
        if self.rot:
            # frequencies in float64; the kernel forms position * f_i exactly, reduces it to [-pi, pi] and takes the float32
            # sine and cosine of that
            i = torch.arange(self.rot // 2, dtype=torch.float64)
            f = torch.pow(torch.tensor(self.base, dtype=torch.float64), -2.0 * i / self.rot) / self.scaling
            self.freq = f.to(device).contiguous()

    def first_weights(self):
        return (self.w_qkv,)

    def cache_need(self):
        return KVNeed(self.nkv, self.dk, None, v_head_dim=self.dv, pool=self.pool)

    def workspace_bytes(self, n_tokens, n_seqs):
        return (nbytes((n_tokens, self.d_qkv), torch.float32) + nbytes((n_tokens, self.nh * self.dk), self.dtype) +
                nbytes((n_tokens, self.nh * self.dv), self.dtype) + nbytes((n_tokens, self.hidden), self.dtype))

    def forward(self, ctx, h, x, cache, accumulate=True):
        h = linear.as_tensor(h)
        T, ws = h.shape[0], ctx.ws
        qkv = ws.alloc((T, self.d_qkv), torch.float32)
        with ctx.prof("qkv_proj"):
            linear.matmul(ctx, h, self.w_qkv, qkv, prefetch=(self.w_o,))
        q = ws.alloc((T, self.nh * self.dk), self.dtype)
        table = ctx.page_table(cache.group)
        with ctx.prof("rope_norm_append"):
            ops.qk_rope_norm_append(qkv, self.b_qkv, q, ctx.tok_pos, ctx.tok_seq, table, cache.k, cache.v, self.nh, self.nkv, self.dk, self.dv,
                                    self.rot, self.freq, self.eps, self.unit_norm, ctx.err)
            if self.pool:
                ops.pool_blocks(ctx.tok_pos, ctx.tok_seq, table, cache.k, cache.v, cache.pooled_k, cache.pooled_v, T, self.nkv, self.dk,
                                self.dv, self.pool, ctx.err)
        a = ws.alloc((T, self.nh * self.dv), self.dtype)
        pooled_k, pooled_v = (cache.pooled_k, cache.pooled_v) if self.pool else (None, None)
        with ctx.prof("attn_window_pooled"):
            if ctx.all_single:      # one token a sequence: a block per (token, head), its warps sharing the keys
                ops.pooled_window_attn(q, a, cache.k, cache.v, pooled_k, pooled_v, ctx.tok_pos, ctx.tok_seq, table, self.nh, self.nkv, self.dk,
                                       self.dv, self.scale, self.window, self.pool)
            else:                   # a prompt step: keys staged once for the 32 rows of a tile
                tiles = ctx.tiles(self.tile_tokens)
                ops.pooled_window_attn_tiled(q, a, cache.k, cache.v, pooled_k, pooled_v, table, tiles.seq, tiles.tok0, tiles.ntok, tiles.pos0,
                                             tiles.count, self.tile_tokens, self.nh, self.nkv, self.dk, self.dv, self.scale, self.window, self.pool)
        with ctx.prof("o_proj"):
            linear.matmul(ctx, a, self.w_o, x, epilogue=linear.EPI_RESIDUAL if accumulate else linear.EPI_STORE,
                          residual=x if accumulate else None, prefetch=ctx.weights_after)
