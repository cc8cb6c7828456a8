"""Attention whose keys and values are expanded from a shared low-rank latent.

Per token the mixer keeps a latent c (size `kv_rank`, RMS-normed with a weight) and one rotated key part (size
`rot_dim`) shared by all heads: [c | k_rot] = W_dkv h.  A query head is [q_n (size `head_dim`) | q_r (size `rot_dim`)];
q_r and k_rot are rotated by position * f_i with half-split pairs (i, i + rot_dim / 2).  Per head the unrotated key is
W_uk c and the value W_uv c, and score = (q_n . W_uk c + q_r . k_rot) * scale.

Since q_n . (W_uk c) = (W_uk^T q_n) . c, the queries are moved into the latent's space once per token and attention
runs over the cache rows [c | k_rot] as they are: one key head of size kv_rank + rot_dim for all query heads, whose first
kv_rank dimensions are also its value; the weighted latents are then expanded with W_uv.  Nothing per head is ever
computed for a cached token.  A prompt step whose sequences all start at position 0 (and which keeps its own latent) sees
only its own tokens: it expands their keys and values per head once, with two matrix products over the rows it has just
written, and attends over those, heads of head_dim + rot_dim against values of v_head_dim, which is several times fewer
multiply-adds than rows of the latent's size.  A layer with `reads_cache` keeps nothing: it has no W_dkv and reads the rows that an
earlier layer of the same kv_rank, rot_dim and rotation left in its cache, with its own W_uk, W_uv, queries and mask.

Angles, the latent's norm, scores, the softmax and the weighted latents are float32 in both precisions; the cache rows
are kept in the compute dtype.
"""
import torch

from ..config.base import ConfigError
from ..csrc import ops
from . import linear
from .base import KVNeed, Part, as_matrix, as_vector, nbytes
from .masked_attention import MASKS, SHARED_KEYS_MIN_GROUP, decode_splits, most_keys, read_mask, single_token_tiles, splits_room
from .registry import register_mixer
from .rope import rotary_frequencies


@register_mixer("latent_attention")
class LatentAttention(Part):
    graph_safe = True

    def __init__(self, spec, env):
        self.hidden = spec["hidden_size"]
        self.nh, self.d, self.rd, self.dv, self.rank = spec["num_heads"], spec["head_dim"], spec["rot_dim"], spec["v_head_dim"], spec["kv_rank"]
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.rot_base, self.rot_scaling = float(spec.get("rot_base") or 10000.0), spec.get("rot_scaling")
        self.reads_foreign_cache = bool(spec.get("reads_cache", False))
        self.names = dict(spec["names"])
        self.dtype = env.dtype
        if self.nh < 1 or self.d < 0 or self.rd < 0 or self.rd % 2 or self.d + self.rd < 1 or self.dv < 1 or self.rank < 1:
            raise ConfigError(f"latent_attention: {self.nh} heads of {self.d} + {self.rd}, values of {self.dv}, a latent of {self.rank}")
        if self.rank + self.rd > 1024 or self.rank > 512:
            raise ConfigError(f"latent_attention: a latent of {self.rank} + {self.rd} is not taken (latent to 512, row to 1024)")
        self.mask, self.mask_size = read_mask(spec.get("mask"), "latent_attention")
        self.dq, self.dc = self.d + self.rd, self.rank + self.rd
        self.d_in = self.nh * self.dq + (0 if self.reads_foreign_cache else self.dc)
        self.tile_tokens = max(1, 32 // self.nh)
        self.freq = self.norm_w = None

    EXPANDED_TILE = 32      # tokens a tile when every head has its own keys (a block's 32 rows are 32 tokens of one head)

    def tile_sizes(self):
        return (self.tile_tokens,) if self.reads_foreign_cache else (self.tile_tokens, self.EXPANDED_TILE)

    def sizes(self):
        return {"heads": self.nh, "head_dim": self.d, "rot_dim": self.rd, "v_head_dim": self.dv, "kv_rank": self.rank,
                "mask": {v: k for k, v in MASKS.items()}[self.mask], "reads_cache": self.reads_foreign_cache}

    def flops(self, n_tokens, attended):
        proj = 2.0 * n_tokens * (self.hidden * (self.d_in + self.nh * self.dv) + self.nh * self.rank * (self.d + self.dv))
        if self.mask != ops.MASK_CAUSAL:
            attended = min(attended, n_tokens * self.mask_size)
        return proj + 2.0 * attended * self.nh * (self.dc + self.rank)

    def weight_shapes(self, prefix):
        n = self.names
        out = {prefix + n["q"]: (self.nh * self.dq, self.hidden), prefix + n["uk"]: (self.nh * self.d, self.rank),
               prefix + n["uv"]: (self.nh * self.dv, self.rank), prefix + n["o"]: (self.hidden, self.nh * self.dv)}
        if not self.reads_foreign_cache:
            out[prefix + n["dkv"]] = (self.dc, self.hidden)
            out[prefix + n["dkv_norm"]] = (self.rank,)
        return out

    def load(self, tensors, prefix, device):
        n = self.names
        mats = [as_matrix(tensors[prefix + n["q"]], self.dtype, device)]
        if not self.reads_foreign_cache:
            mats.append(as_matrix(tensors[prefix + n["dkv"]], self.dtype, device))
            self.norm_w = as_vector(tensors[prefix + n["dkv_norm"]], device)
        self.w_in = torch.cat(mats, dim=0).contiguous()
        # per head: W_uk^T as [rank, d] (queries into the latent's space) and W_uv as [dv, rank] (weighted latents out of it)
        self.w_uk = as_matrix(tensors[prefix + n["uk"]], self.dtype, device)        # [heads * d, rank]: a step's own keys
        self.w_ukt = self.w_uk.view(self.nh, self.d, self.rank).transpose(1, 2).contiguous()
        self.w_uv2 = as_matrix(tensors[prefix + n["uv"]], self.dtype, device)       # [heads * dv, rank]: a step's own values
        self.w_uv = self.w_uv2.view(self.nh, self.dv, self.rank)
        self.w_o = as_matrix(tensors[prefix + n["o"]], self.dtype, device)
        if self.rd:
            self.freq = rotary_frequencies(self.rd, self.rot_base, self.rot_scaling).to(device).contiguous()

    def first_weights(self):
        return (self.w_in,)

    def cache_need(self):
        if self.reads_foreign_cache:
            return None
        return KVNeed(1, self.dc, None, v_head_dim=self.rank, values_in_keys=True)

    def workspace_bytes(self, n_tokens, n_seqs):
        f32 = torch.float32
        absorbed = nbytes((n_tokens, self.nh * self.dc), f32) + nbytes((n_tokens, self.nh * self.rank), f32)
        expanded = (nbytes((n_tokens, self.nh * self.dq), f32) + nbytes((n_tokens, self.dc), self.dtype) + nbytes((n_tokens, self.nh * self.d), self.dtype) +
                    nbytes((n_tokens, self.nh * self.dq), self.dtype) + nbytes((n_tokens, self.nh * self.dv), self.dtype))
        return (nbytes((n_tokens, self.d_in), f32) + max(absorbed + splits_room(n_seqs, self.nh, self.rank), expanded) +
                nbytes((n_tokens, self.nh * self.dv), self.dtype) + nbytes((n_tokens, self.hidden), self.dtype))

    def _forward_own_keys(self, ctx, u, x, cache, accumulate):
        """A prompt step that sees only its own tokens: keys and values expanded per head for the step's tokens."""
        T, ws = u.shape[0], ctx.ws
        q = ws.alloc((T, self.nh * self.dq), torch.float32)
        rows = ws.alloc((T, self.dc), self.dtype)
        table = ctx.page_table(cache.group)
        with ctx.prof("latent_prepare"):
            ops.latent_prepare(u, self.nh * self.dq, True, q, self.dq, self.d, True, self.norm_w, self.eps, ctx.tok_pos, ctx.tok_seq, table,
                               cache.k, self.nh, self.d, self.rd, self.rank, self.freq, ctx.err, row_out=rows)
        kn = ws.alloc((T, self.nh * self.d), self.dtype)
        kx = ws.alloc((T, self.nh * self.dq), self.dtype)
        vx = ws.alloc((T, self.nh * self.dv), self.dtype)
        with ctx.prof("latent_expand"):
            linear.matmul(ctx, rows[:, :self.rank], self.w_uk, kn)
            linear.matmul(ctx, rows[:, :self.rank], self.w_uv2, vx)
            ops.latent_expand_keys(kn, rows, kx, self.nh, self.d, self.rd, self.rank)
        a = ws.alloc((T, self.nh * self.dv), self.dtype)
        tiles = ctx.tiles(self.EXPANDED_TILE)
        with ctx.prof("attn_latent"):
            ops.masked_attn_tiled(q, a, kx, vx, None, tiles.seq, tiles.tok0, tiles.ntok, tiles.pos0, tiles.count, self.EXPANDED_TILE,
                                  self.nh, self.nh, self.dq, self.dv, self.scale, self.mask, self.mask_size, None)
        with ctx.prof("o_proj"):
            linear.matmul(ctx, a, self.w_o, x, epilogue=linear.EPI_RESIDUAL if accumulate else linear.EPI_STORE,
                          residual=x if accumulate else None, prefetch=ctx.weights_after)

    def forward(self, ctx, h, x, cache, accumulate=True):
        h = linear.as_tensor(h)
        T, ws, f32 = h.shape[0], ctx.ws, torch.float32
        if cache is None or cache.k is None or cache.k.shape[-1] != self.dc or cache.v is not None:
            raise ConfigError("latent_attention: the cache entry it was given does not hold rows of its latent's size")
        u = ws.alloc((T, self.d_in), f32)
        with ctx.prof("latent_in_proj"):
            linear.matmul(ctx, h, self.w_in, u, prefetch=(self.w_o,))
        own = not self.reads_foreign_cache
        if own and self.d and not ctx.all_single and ctx.all_fresh:
            return self._forward_own_keys(ctx, u, x, cache, accumulate)
        qf = ws.alloc((T, self.nh * self.dc), f32)
        table = ctx.page_table(cache.group)
        with ctx.prof("latent_prepare"):
            ops.latent_prepare(u, self.nh * self.dq, own, qf, self.dc, self.rank, False, self.norm_w, self.eps, ctx.tok_pos, ctx.tok_seq,
                               table if own else None, cache.k if own else None, self.nh, self.d, self.rd, self.rank, self.freq, ctx.err)
            if self.d:
                ops.head_matmul(u, self.dq, self.w_ukt, qf, self.dc)
            else:
                qf.view(T, self.nh, self.dc)[:, :, :self.rank].zero_()
        ol = ws.alloc((T, self.nh * self.rank), f32)
        with ctx.prof("attn_latent"):
            if ctx.all_single and self.nh >= SHARED_KEYS_MIN_GROUP:     # a row of the latent is staged once for all the heads
                splits = decode_splits(ctx, 1, self.nh, self.mask, self.mask_size)
                part = ws.alloc((T * self.nh * splits * (2 + self.rank),), f32) if splits > 1 else None
                tseq, ttok0, tntok, tpos0 = single_token_tiles(ctx)
                ops.masked_attn_tiled(qf, ol, cache.k, None, table, tseq, ttok0, tntok, tpos0, T, 1, self.nh, 1, self.dc, self.rank, self.scale,
                                      self.mask, self.mask_size, None, n_splits=splits, part=part)
            elif ctx.all_single:
                ops.masked_attn(qf, ol, cache.k, None, ctx.tok_pos, ctx.tok_seq, table, self.nh, 1, self.dc, self.rank, self.scale,
                                self.mask, self.mask_size, None, most_keys(self.mask, self.mask_size))
            else:
                tiles = ctx.tiles(self.tile_tokens)
                ops.masked_attn_tiled(qf, ol, cache.k, None, table, tiles.seq, tiles.tok0, tiles.ntok, tiles.pos0, tiles.count,
                                      self.tile_tokens, self.nh, 1, self.dc, self.rank, self.scale, self.mask, self.mask_size, None)
        a = ws.alloc((T, self.nh * self.dv), self.dtype)
        with ctx.prof("latent_values"):
            ops.head_matmul(ol, self.rank, self.w_uv, a, self.dv)
        with ctx.prof("o_proj"):
            linear.matmul(ctx, a, self.w_o, x, epilogue=linear.EPI_RESIDUAL if accumulate else linear.EPI_STORE,
                          residual=x if accumulate else None, prefetch=ctx.weights_after)
