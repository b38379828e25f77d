"""Grouped-query attention over the paged cache.

q = h Wq^T + bq, k = h Wk^T + bk, v = h Wv^T + bv (one fused product over the
stacked weights); q and k are rotated at their absolute positions; k (after the
rotation) and v are written into the cache pages of their request; every row
then attends to the keys of its request up to its own position (inside the
window, where the layer has one: a key is hidden when key + window < query),
scores q.k / sqrt(head_dim) with the scale applied after the product, softmax
in float32; kv head g serves query heads g*n .. (g+1)*n - 1; the merged heads go
through Wo (reference: qwen-infer/src/model.rs:262-328, 397-414, 119-129).
"""
from __future__ import annotations

import math
import os

import numpy as np
import torch

from ..config.spec import ConfigError
from ..kernels import ops
from ..weights.store import TensorSpec
from .base import BatchAnnotation, CacheNeed, KVNeed, build_part, register_part
from . import gemm_bf16
from .linear import Linear

_position_tables = {}

# Which kernel takes long prompt portions in bfloat16: the tcgen05 kernel (128-row
# tiles, scores and outputs in tensor memory; 45 us on 2,048 tokens of 14 heads) or,
# with TOKB200_ATTENTION=mma, the mma.sync kernel (64-row tiles; 73 us), which also
# takes the short portions and the head sizes the first does not.
_PROMPT_KERNEL = os.environ.get("TOKB200_ATTENTION", "tcgen05")
# TOKB200_QKV_NORM=separate keeps the norm in front of the projection of few rows a kernel of its own
# TOKB200_QKV_ROPE=fused folds rotation and cache write of many rows into the tcgen05 product's
# epilogue.  With one tile a block the longer epilogue is not hidden behind other tiles, and it
# costs what the separate kernel costs (3.27 against 3.26 ms for 2,048 tokens), so it is off
# unless asked for.
_FUSED_QKV = os.environ.get("TOKB200_QKV_ROPE", "separate") == "fused"
_FUSED_NORM = os.environ.get("TOKB200_QKV_NORM", "fused") != "separate"
# TOKB200_LAYER=fused runs a decoding step's layer (up to 32 rows) as ONE kernel instead of four
# (projection, attention, output projection, feed-forward).  It is correct and off by default:
# measured at 36 us a layer against 27 us for the four kernels (8 rows, Qwen2.5-0.5B sizes),
# because its phases run one after the other behind barriers over all blocks, each a chain of
# two or three trips to L2, while the four kernels overlap their heads and tails.  The
# switches that take the norm or the feed-forward out of their fusions turn it off as well.
_FUSED_LAYER = os.environ.get("TOKB200_LAYER", "separate") == "fused" and _FUSED_NORM


class RowTiles(BatchAnnotation):
    """The step's rows cut into tiles of up to `rows` consecutive rows of one request, as the
    prompt-attention kernels take them: int32 [tiles, 2] = (first row, rows), the tile that
    walks the most keys first (the kernels place blocks in that order, so the longest work
    starts first).  Unused tiles of a padded step have no rows.  With `long_only`, requests
    that bring a single token get no tile when others bring more (their rows are `SingleRows`',
    served by the decoding kernel: a tile of one row would walk its keys at a tile's cost)."""

    def __init__(self, rows: int, long_only: bool = False):
        self.rows = rows
        self.long_only = long_only
        self.key = f"row_tiles_{rows}" + ("_long" if long_only else "")

    def capacity(self, n_tokens, n_requests):
        return 2 * (n_tokens // self.rows + n_requests)

    def fill(self, out, first_rows, counts, starts, padded):
        n = len(counts)
        if self.long_only and n and int(counts.max()) > 1:
            keep = counts > 1
            first_rows, counts, starts = first_rows[keep], counts[keep], starts[keep]
            n = len(counts)
        if n and int(counts.max()) == 1:
            # one tile of one row a request: a stable order, as a sort of tuples gives
            order = np.argsort(-starts, kind="stable")
            out[0:2 * n:2] = first_rows[order]
            out[1:2 * n:2] = 1
            made = n
        else:
            tiles = []    # (last position + 1: the keys the tile walks, first row, rows)
            for first_row, count, start in zip(first_rows.tolist(), counts.tolist(), starts.tolist()):
                for first in range(0, count, self.rows):
                    here = min(self.rows, count - first)
                    tiles.append((start + first + here, first_row + first, here))
            tiles.sort(key=lambda item: -item[0])
            for at, (_, first_row, here) in enumerate(tiles):
                out[2 * at] = first_row
                out[2 * at + 1] = here
            made = len(tiles)
        return len(out) // 2 if padded else made

    def view(self, words):
        return words.view(-1, 2)


class SingleRows(BatchAnnotation):
    """The rows of requests that bring exactly one token, when the step also brings portions
    of others: int32 [requests], row indices, -1 where there is none.  A step of single tokens
    alone has none (all of its rows go to the decoding kernel anyway)."""

    key = "single_rows"

    def capacity(self, n_tokens, n_requests):
        return n_requests

    def fill(self, out, first_rows, counts, starts, padded):
        out[:] = -1
        made = 0
        if len(counts) and int(counts.max()) > 1:
            rows = first_rows[counts == 1]
            out[:len(rows)] = rows
            made = len(rows)
        # a captured step keeps the launch for as many rows as it has requests, but only a step
        # that has such rows at all: steps of portions alone are captured without it (their key
        # differs, see Attention.shape_key)
        return (len(out) if made else 0) if padded else made


# the tiles of the two prompt kernels: 64 rows (mma.sync) and 128 rows (tcgen05), for all
# requests and for those alone that bring more than one token
_TILES = RowTiles(ops.PREFILL_TILE_ROWS)
_WIDE_TILES = RowTiles(ops.WIDE_TILE_ROWS)
_LONG_TILES = RowTiles(ops.PREFILL_TILE_ROWS, long_only=True)
_LONG_WIDE_TILES = RowTiles(ops.WIDE_TILE_ROWS, long_only=True)
_SINGLES = SingleRows()
# TOKB200_MIXED=tiles sends the single-token rows of a mixed step through the kernels for portions
_SPLIT_MIXED = os.environ.get("TOKB200_MIXED", "split") != "tiles"
# portions from this length on go to the tcgen05 kernel (shorter ones would leave most of a
# 128-row tile empty)
_WIDE_FROM = 96


class PagedAttention:
    """What every mixer that attends over the paged cache shares: the annotations its kernels
    want packed with a step, the kernel choice (`attend`) and its say in a captured step's key.
    A mixer that inherits it sets `nh` (query heads), `nkv` (heads of the cache rows), `d` (lanes
    of a cache row's head), `window` (None: all keys), `chunk` (None: no chunks), `scale` and, where its softmax has one,
    `sink` (float32, one learned score per query head that counts once in the denominator) and `softcap` (scores squashed
    into (-softcap, softcap) by a tanh)."""

    graph_safe = True   # launches depend on device-side metadata only
    sink = None
    chunk = None        # n: keys are seen inside chunks of n positions counted from 0
    softcap = None      # c: a score s counts as c * tanh(s / c)

    def batch_annotations(self):
        return [_TILES, _WIDE_TILES, _LONG_TILES, _LONG_WIDE_TILES, _SINGLES]

    def shape_key(self, q_lens):
        """Which attention kernel a step of these portion lengths gets (part of the key under
        which the engine keeps a captured step)."""
        longest = max(q_lens) if q_lens else 0
        if longest == 1:
            return "single"
        kind = "wide" if longest >= _WIDE_FROM else "tiles"
        # portions with single tokens beside them launch the decoding kernel too
        return kind + "+1" if min(q_lens) == 1 else kind

    def attend(self, q, out, ctx, group, cache):
        """Choose the kernel by precision and by the shape of the batch.  A group that keeps one
        row a token (`cache.v_pool` None) is read as keys and as values: the values are then the
        leading lanes of the key rows, and `out` has the key rows' width."""
        k_pool = cache.k_pool
        v_pool = cache.v_pool if cache.v_pool is not None else cache.k_pool
        sink = self.sink
        if q.dtype == torch.bfloat16 and ctx.max_q_len == 1 and \
                ops.decode_attention_supported(self.nh, self.nkv, self.d):
            ops.decode_attention(
                q, k_pool, v_pool, out, group.block_table, ctx.row_req, ctx.pos,
                self.nh, self.nkv, self.d, group.page_size, self.window, self.scale, sink=sink, chunk=self.chunk, softcap=self.softcap)
            return
        wide, tiles = ctx.views.get(_WIDE_TILES.key), ctx.views.get(_TILES.key)
        singles = ctx.views.get(_SINGLES.key)
        if _SPLIT_MIXED and q.dtype == torch.bfloat16 and singles is not None and singles[1] > 0 and \
                ops.decode_attention_supported(self.nh, self.nkv, self.d) and \
                ctx.views.get(_LONG_WIDE_TILES.key) is not None and ctx.views.get(_LONG_TILES.key) is not None:
            # a step of portions AND single tokens: the single-token rows go to the decoding kernel
            # (keys split over blocks, the group's heads as one tile), the portions to theirs
            ops.decode_attention(
                q, k_pool, v_pool, out, group.block_table, ctx.row_req, ctx.pos,
                self.nh, self.nkv, self.d, group.page_size, self.window, self.scale, rows=singles[0], sink=sink, chunk=self.chunk, softcap=self.softcap)
            wide, tiles = ctx.views[_LONG_WIDE_TILES.key], ctx.views[_LONG_TILES.key]
        if _PROMPT_KERNEL == "tcgen05" and q.dtype == torch.bfloat16 and \
                wide is not None and ctx.max_q_len >= _WIDE_FROM and \
                ops.attention_tcgen05_supported(self.nh, self.nkv, self.d):
            # long portions on the tcgen05 kernel (128-row tiles, scores in tensor memory)
            ops.attention_tcgen05(
                q, k_pool, v_pool, out, group.block_table, ctx.row_req, ctx.pos,
                wide[0], wide[1], self.nh, self.nkv, self.d, group.page_size,
                self.window, self.scale, sink=sink, chunk=self.chunk, softcap=self.softcap)
            return
        if q.dtype == torch.bfloat16 and tiles is not None and \
                ops.prefill_attention_supported(self.nh, self.nkv, self.d):
            ops.prefill_attention(
                q, k_pool, v_pool, out, group.block_table, ctx.row_req, ctx.pos,
                tiles[0], tiles[1], self.nh, self.nkv, self.d, group.page_size,
                self.window, self.scale, sink=sink, chunk=self.chunk, softcap=self.softcap)
            return
        ops.paged_attention_generic(
            q, k_pool, v_pool, out, group.block_table, ctx.row_req, ctx.pos,
            self.nh, self.nkv, self.d, group.page_size, self.window, self.scale, sink=sink, chunk=self.chunk, softcap=self.softcap)


class GQAttention(PagedAttention):
    @staticmethod
    def tensors(spec):
        p, x = spec.params, spec.prefix
        q_out, kv_out = p["num_heads"] * p["head_dim"], p["num_kv_heads"] * p["head_dim"]
        out = [
            TensorSpec(x + ".q_proj.weight", (q_out, p["hidden_size"])),
            TensorSpec(x + ".k_proj.weight", (kv_out, p["hidden_size"])),
            TensorSpec(x + ".v_proj.weight", (kv_out, p["hidden_size"])),
            TensorSpec(x + ".o_proj.weight", (p["hidden_size"], q_out)),
        ]
        if p.get("qkv_bias"):
            out += [TensorSpec(x + ".q_proj.bias", (q_out,)),
                    TensorSpec(x + ".k_proj.bias", (kv_out,)),
                    TensorSpec(x + ".v_proj.bias", (kv_out,))]
        if p.get("out_bias"):
            out.append(TensorSpec(x + ".o_proj.bias", (p["hidden_size"],)))
        return out

    def __init__(self, spec, store, runtime):
        p, x = spec.params, spec.prefix
        self.runtime = runtime
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.d = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        self.window = p.get("window")
        if self.nh % self.nkv:
            raise ConfigError(f"{self.nh} query heads is not a multiple of {self.nkv} kv heads")
        if self.d % 2:
            raise ConfigError(f"head size {self.d} must be even")
        self.scale = 1.0 / math.sqrt(float(self.d))
        # one stacked product for q, k and v
        w_qkv = torch.cat([store.get(x + f".{n}_proj.weight") for n in "qkv"], dim=0)
        self.qkv = Linear(runtime.matrix(w_qkv))
        self.qkv_bias = None
        if p.get("qkv_bias"):
            self.qkv_bias = runtime.vector(
                torch.cat([store.get(x + f".{n}_proj.bias").to(torch.float32) for n in "qkv"]))
        self.out = Linear(
            runtime.matrix(store.get(x + ".o_proj.weight")),
            runtime.vector(store.get(x + ".o_proj.bias")) if p.get("out_bias") else None)
        # layers with the same position constants share one table
        pos_spec = p["position"]
        key = (pos_spec.kind, tuple(sorted(pos_spec.params.items())), str(runtime.device))
        if key not in _position_tables:
            _position_tables[key] = build_part("position", pos_spec, store, runtime)
        self.position = _position_tables[key]
        if self.position.rotary_dim > self.d:
            raise ConfigError("the rotary width exceeds the head size")

    def cache_need(self):
        return CacheNeed(kv=KVNeed(self.nkv, self.d, self.window))

    def streamed_weights(self):
        return [self.qkv.weight, self.out.weight]

    def start_operands(self):
        """(first weight, its bias): what this mixer's first kernel reads."""
        return self.qkv.weight, self.qkv_bias

    def fused_layer(self, stream, norm, ctx, cache, feed_forward, feed_forward_norm) -> bool:
        """For a step of few rows of one token each in bfloat16: the WHOLE pre-norm layer in one
        kernel (both norms, this attention, a gated feed-forward), straight from the stream.
        The norms must offer `folded() -> (gain, eps)` of an RMS norm and the feed-forward
        `gated_operands() -> (interleaved gate/up weight, down weight, activation)`.  True when it
        was done: the stream then holds the sum after the attention, and the feed-forward's output
        as pending partial sums.  False: the block runs the parts one by one."""
        fold, fold2 = getattr(norm, "folded", None), getattr(feed_forward_norm, "folded", None)
        operands = getattr(feed_forward, "gated_operands", None)
        x = stream.x
        if not (_FUSED_LAYER and fold is not None and fold2 is not None and operands is not None and
                self.runtime.dtype == torch.bfloat16 and ctx.max_q_len == 1 and self.out.bias is None and
                self.position.rotary_dim == self.d and cache.k_pool is not None):
            return False
        gated = operands()
        if gated is None:
            return False
        w_gate_up, w_down, activation = gated
        down_splits, _ = ops.layer_small_m_splits(x.shape[0], self.hidden, w_down.shape[1], self.nh, self.nkv, self.d)
        if down_splits == 0:
            return False
        (gain1, eps1), (gain2, eps2) = fold(), fold2()
        group = ctx.groups[cache.group]
        delta, stream.pending = stream.pending, None
        x_mid, x_out = torch.empty_like(x), torch.empty_like(x)
        out = torch.empty((down_splits,) + tuple(x.shape), dtype=torch.float32, device=x.device)
        ahead = getattr(ctx.next_block, "layer_start_operands", None)
        ops.layer_small_m(x, delta, x_mid, x_out, out, gain1, eps1, self.qkv.weight, self.qkv_bias, ctx.pos,
                          group.slots, ctx.row_req, group.block_table, self.position.cos, self.position.sin,
                          cache.k_pool, cache.v_pool, cache.writes, self.out.weight, gain2, eps2, w_gate_up,
                          w_down, self.nh, self.nkv, self.d, group.page_size, self.window, self.scale, activation,
                          next_layer=ahead() if ahead is not None else None)
        stream.x, stream.pending = x_out, out
        return True

    def fused_step(self, stream, norm, ctx, cache):
        """For few rows in bfloat16: the residual add and the norm in front are computed by
        the projection kernel itself, straight from the stream (the norm must offer
        `folded() -> (gain, eps)` of an RMS norm).  Returns this part's output, or None when
        the sizes are not taken (the block then norms and calls `forward`)."""
        fold = getattr(norm, "folded", None)
        x = stream.x
        if not (_FUSED_NORM and fold is not None and self.runtime.dtype == torch.bfloat16 and
                ops.qkv_norm_rope_small_m_supported(x.shape[0], self.hidden, self.d,
                                                    self.position.rotary_dim)):
            return None
        gain, eps = fold()
        group = ctx.groups[cache.group]
        delta, stream.pending = stream.pending, None
        x_out = torch.empty_like(x)
        q = self.runtime.empty(ctx.n_tokens, self.nh * self.d)
        ops.qkv_norm_rope_small_m(
            x, x_out, delta, gain, eps, self.qkv.weight, self.qkv_bias, ctx.pos,
            group.slots if cache.writes else None, self.position.cos, self.position.sin, q,
            cache.k_pool if cache.writes else None, cache.v_pool if cache.writes else None,
            self.nh, self.nkv, self.d)
        stream.x = x_out
        mixed = self.runtime.empty(ctx.n_tokens, self.nh * self.d)
        self.attend(q, mixed, ctx, group, cache)
        return self.out.forward(mixed, partials_ok=True)

    def forward(self, h, ctx, cache):
        q = self.runtime.empty(ctx.n_tokens, self.nh * self.d)
        group = ctx.groups[cache.group]
        if h.dtype == torch.bfloat16 and ops.qkv_rope_small_m_supported(
                h.shape[0], self.hidden, self.d, self.position.rotary_dim, self.qkv.out_features):
            # few rows: projection, bias, rotation and cache write in one kernel
            ops.qkv_rope_small_m(
                h, self.qkv.weight, self.qkv_bias, ctx.pos, group.slots if cache.writes else None,
                self.position.cos, self.position.sin, q,
                cache.k_pool if cache.writes else None, cache.v_pool if cache.writes else None,
                self.nh, self.nkv, self.d)
            mixed = self.runtime.empty(ctx.n_tokens, self.nh * self.d)
            self.attend(q, mixed, ctx, group, cache)
            return self.out.forward(mixed, partials_ok=True)
        if h.dtype == torch.bfloat16 and _FUSED_QKV and \
                gemm_bf16.choose_tile_k_splits(h.shape[0], self.qkv.out_features, self.hidden) == 1 and \
                gemm_bf16.use_tcgen05(h.shape[0], self.qkv.out_features, self.hidden) and \
                ops.gemm_qkv_rope_supported(self.hidden, self.nh, self.nkv, self.d, self.position.rotary_dim):
            # many rows: the tcgen05 product with bias, rotation and cache write in its epilogue
            ops.gemm_qkv_rope(
                h, self.qkv.weight, self.qkv_bias, ctx.pos, group.slots if cache.writes else None,
                self.position.cos, self.position.sin, q,
                cache.k_pool if cache.writes else None, cache.v_pool if cache.writes else None,
                self.nh, self.nkv, self.d)
            mixed = self.runtime.empty(ctx.n_tokens, self.nh * self.d)
            self.attend(q, mixed, ctx, group, cache)
            return self.out.forward(mixed, partials_ok=True)
        # in bfloat16 with a whole-head rotation the product may come as partial sums over k
        # (a few dozen rows and a narrow matrix fill the device only that way)
        sums_ok = h.dtype == torch.bfloat16 and self.position.rotary_dim == self.d and self.d % 16 == 0
        qkv = self.qkv.forward(h, partials_ok=sums_ok)
        ops.rope_store(
            qkv, self.qkv_bias, ctx.pos, group.slots if cache.writes else None,
            self.position.cos, self.position.sin, q,
            cache.k_pool if cache.writes else None, cache.v_pool if cache.writes else None,
            self.nh, self.nkv, self.d, self.position.rotary_dim)
        mixed = self.runtime.empty(ctx.n_tokens, self.nh * self.d)
        self.attend(q, mixed, ctx, group, cache)
        return self.out.forward(mixed, partials_ok=True)


class RotaryGQAttention(PagedAttention):
    """Grouped-query attention whose key and value heads may differ in size, with biases, a score
    scale of its own and the interleaved rotation on the leading lanes of every query and key head:
    q = Wq h + bq (heads x dim), k = Wk h + bk (kv_heads x dim), v = Wv h + bv (kv_heads x vdim);
    score = q . k * scale; softmax over the keys the query sees (all earlier ones, those inside
    `window`, or those of its own chunk of `chunk` positions counted from the sequence's start);
    Wo on the heads' outputs (heads x vdim).  Tensors `<prefix>.q`, `.k`, `.v` (+ `.b` with
    `bias`), `.o`.

    Cache rows and query rows have `row` lanes a head, max(dim, vdim) rounded up to whole 16s: keys
    and queries fill the first dim lanes, values the first vdim, zeros behind (a zero lane adds
    nothing to a score; a zero value lane meets a zero column of the padded Wo), so that the paged
    kernels, which take one head size, serve both.  `input_stack` / `forward_projected` as for
    the other mixers that may run side by side.

    More parameters, each off unless given: `qk_norm` (the whole q and the whole k projection divided by their
    root mean square, with gains `.q.norm`, `.k.norm`), `head_temperature`, `sink`; the rotation's layout comes
    with its `position` part (interleaved pairs or halves); `head_norm` (after the rotation every query and key
    head is divided by its root mean square over dim, `norm_eps` inside the root, no gain); `softcap` (a score s
    counts as softcap * tanh(s / softcap)); `output_gate` (the heads' outputs are multiplied by sigmoid(Wg h),
    tensor `.g`, heads * vdim rows; the product rides in the stacked input product); `own_kv` False (the layer
    has no k and v tensors and is called on an earlier call's cache: it projects, rotates and norms queries
    only); `cache_chunk` (what the cache manager may give back, where other calls read this cache with chunks of
    their own: a chunk size that all of theirs divide, or None to keep every page)."""

    @staticmethod
    def tensors(spec):
        p, x = spec.params, spec.prefix
        hidden, heads, groups, dim, vdim = p["hidden_size"], p["heads"], p["kv_heads"], p["dim"], p["vdim"]
        own = p.get("own_kv", True)
        out = [TensorSpec(x + ".q", (heads * dim, hidden))]
        if own:
            out += [TensorSpec(x + ".k", (groups * dim, hidden)), TensorSpec(x + ".v", (groups * vdim, hidden))]
        out.append(TensorSpec(x + ".o", (hidden, heads * vdim)))
        if p.get("bias", True):
            out.append(TensorSpec(x + ".q.b", (heads * dim,)))
            if own:
                out += [TensorSpec(x + ".k.b", (groups * dim,)), TensorSpec(x + ".v.b", (groups * vdim,))]
        if p.get("qk_norm"):
            out.append(TensorSpec(x + ".q.norm", (heads * dim,), "one_plus_normal", 0.1))
            if own:
                out.append(TensorSpec(x + ".k.norm", (groups * dim,), "one_plus_normal", 0.1))
        if p.get("output_gate"):
            out.append(TensorSpec(x + ".g", (heads * vdim, hidden)))
        if p.get("head_temperature"):
            out.append(TensorSpec(x + ".temp", (heads,), "one_plus_normal", 0.2))
        if p.get("sink"):
            out.append(TensorSpec(x + ".sink", (heads,), "normal", 1.0))
        return out

    def __init__(self, spec, store, runtime):
        p, x = spec.params, spec.prefix
        self.runtime = runtime
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.scale = float(p["scale"])
        self.window, self.chunk = p.get("window"), p.get("chunk")
        self.softcap = float(p["softcap"]) if p.get("softcap") is not None else None
        self.own_kv = bool(p.get("own_kv", True))
        self.cache_chunk = p["cache_chunk"] if "cache_chunk" in p else self.chunk
        self.head_norm = bool(p.get("head_norm"))
        if self.softcap is not None and self.softcap <= 0:
            raise ConfigError("a cap on the scores is positive")
        if self.nkv <= 0 or self.nh % self.nkv:
            raise ConfigError(f"{self.nh} query heads is not a multiple of {self.nkv} kv heads")
        if self.chunk is not None and int(self.chunk) < 1:
            raise ConfigError("a chunk holds at least one position")
        self.row = -(-max(self.dim, self.vdim) // 16) * 16
        self.d = self.row
        self.position, self.rot_dims = None, 0
        if p.get("position") is not None:
            self.position = build_part("position", p["position"], store, runtime)
            self.rot_dims = int(self.position.dims)
            if self.rot_dims > self.dim:
                raise ConfigError(f"{self.rot_dims} rotated lanes do not fit a head of {self.dim}")
        names = "qkv" if self.own_kv else "q"
        self._stack = [store.get(x + "." + n) for n in names]
        # the gate's pre-activations are more columns of the stacked product, behind q, k and v
        self.gate_at = None
        if p.get("output_gate"):
            self.gate_at = sum(w.shape[0] for w in self._stack)
            self._stack.append(store.get(x + ".g"))
        self.bias = None
        if p.get("bias", True):
            self.bias = runtime.vector(torch.cat([store.get(x + f".{n}.b").to(torch.float32) for n in names]))
        self.q_gain = self.k_gain = self.temp = None
        self.norm_eps = float(p.get("norm_eps", 0.0))
        if p.get("qk_norm"):
            self.q_gain = runtime.vector(store.get(x + ".q.norm"))
            if self.own_kv:
                self.k_gain = runtime.vector(store.get(x + ".k.norm"))
        if p.get("head_temperature"):
            self.temp = runtime.vector(store.get(x + ".temp"))
        if p.get("sink"):
            self.sink = runtime.vector(store.get(x + ".sink"))
        w_o = store.get(x + ".o")
        if self.row != self.vdim:           # zero columns where the value lanes end
            wide = torch.zeros((self.hidden, self.nh, self.row), dtype=w_o.dtype)
            wide[:, :, :self.vdim] = w_o.view(self.hidden, self.nh, self.vdim)
            w_o = wide.view(self.hidden, self.nh * self.row)
        self.out = Linear(runtime.matrix(w_o))
        self.inputs = None

    def input_stack(self):
        """(q, k and v matrices one under the other, as stored; nothing of their bias: the kernel
        that rotates adds it)."""
        return torch.cat(self._stack, dim=0), None

    def cache_need(self):
        return CacheNeed(kv=KVNeed(self.nkv, self.row, self.window, chunk=self.cache_chunk))

    def streamed_weights(self):
        return [self.out.weight] if self.inputs is None else [self.inputs.weight, self.out.weight]

    def forward_projected(self, proj, at, ctx, cache, out_scale: float = 1.0):
        if out_scale != 1.0:
            raise ValueError("this mixer's output is scaled by whoever adds it")
        if self.own_kv != cache.writes:
            raise ValueError("a layer with keys of its own writes its cache; one without reads an earlier call's")
        group = ctx.groups[cache.group]
        q = self.runtime.empty(ctx.n_tokens, self.nh * self.row)
        ops.qkv_rotate_store(proj, at, self.bias, self.position.inv_freq64 if self.position is not None else None,
                             self.rot_dims, ctx.pos, group.slots if cache.writes else None, ctx.row_req, q,
                             cache.k_pool if self.own_kv else None, cache.v_pool if self.own_kv else None, self.nh,
                             self.nkv if self.own_kv else 0, self.dim, self.vdim, self.row,
                             q_gain=self.q_gain, k_gain=self.k_gain, eps=self.norm_eps, temp=self.temp,
                             layout=getattr(self.position, "layout", "interleaved"),
                             head_norm_eps=self.norm_eps if self.head_norm else None)
        mixed = self.runtime.empty(ctx.n_tokens, self.nh * self.row)
        self.attend(q, mixed, ctx, group, cache)
        if self.gate_at is not None:
            ops.attention_gate(mixed, proj, at + self.gate_at, self.nh, self.vdim, self.row)
        return self.out.forward(mixed, partials_ok=True)

    def forward(self, h, ctx, cache):
        if self.inputs is None:
            from .recurrent import stacked_rows
            self.inputs = Linear(self.runtime.matrix(stacked_rows([self.input_stack()[0]])))
        return self.forward_projected(self.inputs.forward(h, out_dtype=torch.float32), 0, ctx, cache)


register_part("mixer", "gqa_attention", GQAttention)
register_part("mixer", "gqa_rotary", RotaryGQAttention)
