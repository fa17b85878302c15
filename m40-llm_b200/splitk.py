"""Multi-GPU plumbing of the decode path: one process per GPU, `torch.distributed` for the exchange.

Two ways the path shards (one 8-GPU box):

* batched variable-length decode: independent sequences are dealt to ranks (`shard_sequences`); no data-path
  collective at all;
* one long sequence, split-K: every rank owns a contiguous range of the sequence's KV blocks, computes an
  unnormalised (max, sum, out) triple per q head over its range and the triples are all-gathered and merged. With
  the compressed cache (FP16 K / q4 V, top-k block selection) there is one more exchange before that: every rank
  scores its own blocks, keeps its local top-k as (score, block) pairs and the pairs are all-gathered, so that every
  rank derives the same global top-k list (same rule, ties to the lower block).

The exchange payloads are tiny (Qwen2.5-3B shape at 32K context: 16 heads x 64 pairs = 8 KB per rank; triples 16 x 130
floats = 8 KB per rank), so they go through the library collective (NCCL over NVLink on GPUs, gloo on CPU ranks).
Gathered data always lands in the receiving rank's own memory before a kernel reads it. On GPUs the whole chain
(scores, local top-k, all-gather, global top-k, attention, all-gather, merge) is enqueued on the context's decode
stream with no host synchronisation in between (`DeviceSplitK`).

The compute legs are callables so that the same orchestration runs over the CUDA entry points (`NativeLegs`, the
product) and over any other implementation of the legs (the CPU tests pass a numpy restatement and run two gloo
ranks). Nothing here falls back to a CPU computation by itself.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, Sequence

import numpy as np
import torch
import torch.distributed as dist

EMPTY_BLOCK = 0xFFFFFFFF
MAX_TOP_BLOCKS = 64          # slots per q head in a block list (the reference's cap, cuda/kernels.cu:2861-2930)
SCORE_FLOOR = -1.0e30        # scores at or below this are never selected


# ----------------------------------------------------------------------------- plans (pure host logic)
def block_ranges(n_blocks: int, world: int) -> list[tuple[int, int]]:
    """Contiguous, balanced block ranges [begin, end) for ranks 0..world-1 (sizes differ by at most one,
    larger ranges first; ranks beyond n_blocks get empty ranges)."""
    if n_blocks < 0 or world <= 0:
        raise ValueError("n_blocks must be >= 0 and world > 0")
    base, extra = divmod(n_blocks, world)
    out, b = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append((b, b + n))
        b += n
    return out


def token_ranges(seq_len: int, world: int, align: int = 64) -> list[tuple[int, int]]:
    """Token ranges for dense split-K: whole `align`-token tiles per rank, the ragged tail on the last non-empty
    rank."""
    tiles = (seq_len + align - 1) // align
    return [(min(b * align, seq_len), min(e * align, seq_len)) for b, e in block_ranges(tiles, world)]


def shard_sequences(context_lens: Sequence[int], world: int, max_per_rank: int | None = None) -> list[list[int]]:
    """Deals independent sequences to ranks, longest first onto the least-loaded rank (decode attention cost is
    linear in context length). `max_per_rank` caps the number of sequences a rank takes (the projections cost per
    row, so a scheduler keeps row counts equal while balancing tokens); full ranks are skipped. Returns the sequence
    indices of every rank, each list in ascending order."""
    if world <= 0:
        raise ValueError("world must be > 0")
    if max_per_rank is not None and max_per_rank * world < len(context_lens):
        raise ValueError("max_per_rank * world is smaller than the number of sequences")
    loads = [0] * world
    out: list[list[int]] = [[] for _ in range(world)]
    order = sorted(range(len(context_lens)), key=lambda i: (-int(context_lens[i]), i))
    for i in order:
        open_ranks = [j for j in range(world) if max_per_rank is None or len(out[j]) < max_per_rank]
        r = min(open_ranks, key=lambda j: (loads[j], j))
        out[r].append(i)
        loads[r] += int(context_lens[i])
    return [sorted(s) for s in out]


def select_global_topk(scores: np.ndarray, top_blocks: int) -> np.ndarray:
    """Global block list per q head from the gathered scores [q_heads, n_blocks] (f32): the `top_blocks` highest
    scores in descending order, ties to the lower block index, NaN and scores <= -1e30 never selected, unused
    slots EMPTY_BLOCK. Same rule as the single-GPU selection (cuda/kernels.cu:2861-2930, 6526-6600), so every rank
    derives the identical list without a further exchange."""
    if not 1 <= top_blocks <= MAX_TOP_BLOCKS:
        raise ValueError(f"top_blocks must be in 1..{MAX_TOP_BLOCKS}")
    scores = np.asarray(scores, dtype=np.float32)
    q_heads, nb = scores.shape
    out = np.full((q_heads, MAX_TOP_BLOCKS), EMPTY_BLOCK, dtype=np.uint32)
    for h in range(q_heads):
        s = scores[h]
        ok = np.flatnonzero(~np.isnan(s) & (s > np.float32(SCORE_FLOOR)))
        # stable sort of the negated scores keeps the lower index first among equals
        order = ok[np.argsort(-s[ok], kind="stable")][:top_blocks]
        out[h, :order.size] = order.astype(np.uint32)
    return out


def merge_triples(m: np.ndarray, l: np.ndarray, o: np.ndarray) -> np.ndarray:
    """Host statement of the merge the device kernel performs (for plans and tests; the product merges on the
    GPU): m, l [parts, heads], o [parts, heads, hd] unnormalised -> out [heads * hd]. Parts with l == 0 are
    empty."""
    m = np.asarray(m, np.float32)
    l = np.asarray(l, np.float32)
    o = np.asarray(o, np.float32)
    live = l > 0
    mm = np.where(live, m, -np.inf).max(axis=0)                       # [heads]
    w = np.where(live, np.exp((m - mm[None, :]).astype(np.float32)), np.float32(0))
    den = (w * l).sum(axis=0)
    num = (w[:, :, None] * o).sum(axis=0)
    out = np.where(den[:, None] > 0, num / np.maximum(den[:, None], np.float32(1e-38)), np.float32(0))
    return out.astype(np.float32).reshape(-1)


# ----------------------------------------------------------------------------- exchange
def _world(group) -> tuple[int, int]:
    return dist.get_rank(group), dist.get_world_size(group)


def gather_scores(local: torch.Tensor, ranges: Sequence[tuple[int, int]], group=None) -> torch.Tensor:
    """All-gathers the per-rank score slabs [q_heads, end-begin] into the full [q_heads, n_blocks] matrix on every
    rank. Slabs are padded to the widest range so that one fixed-size all-gather does it."""
    rank, world = _world(group)
    q_heads = local.shape[0]
    widest = max(max(e - b for b, e in ranges), 1)
    b, e = ranges[rank]
    assert local.shape == (q_heads, e - b), (tuple(local.shape), ranges[rank])
    send = torch.full((q_heads, widest), float("-inf"), dtype=torch.float32, device=local.device)
    send[:, :e - b] = local
    # output = the ranks' slabs concatenated along dim 0 (the form both NCCL and gloo accept)
    recv = torch.empty((world * q_heads, widest), dtype=torch.float32, device=local.device)
    dist.all_gather_into_tensor(recv, send, group=group)
    recv = recv.view(world, q_heads, widest)
    n_blocks = ranges[-1][1]
    full = torch.empty((q_heads, n_blocks), dtype=torch.float32, device=local.device)
    for r, (rb, re) in enumerate(ranges):
        full[:, rb:re] = recv[r, :, :re - rb]
    return full


def gather_triples(m: torch.Tensor, l: torch.Tensor, o: torch.Tensor, group=None):
    """All-gathers one rank's triples (m, l [heads]; o [heads, hd]) as ONE message per rank; returns
    (m [world, heads], l [world, heads], o [world, heads, hd]), each contiguous."""
    _, world = _world(group)
    heads, hd = o.shape
    send = torch.cat([m.reshape(heads, 1), l.reshape(heads, 1), o], dim=1).contiguous()
    recv = torch.empty((world * heads, hd + 2), dtype=torch.float32, device=o.device)
    dist.all_gather_into_tensor(recv, send, group=group)
    recv = recv.view(world, heads, hd + 2)
    return recv[:, :, 0].contiguous(), recv[:, :, 1].contiguous(), recv[:, :, 2:].contiguous()


# ----------------------------------------------------------------------------- orchestration
@dataclass
class Legs:
    """The compute legs of one rank. `score(b0, b1) -> [q_heads, b1-b0]` f32 tensor; `topk_pairs(scores, b0, top) ->
    [q_heads, 64, 2]` f32 tensor of (score, block-id bits) pairs; `merge_pairs(pairs [world, q_heads, 64, 2], top) ->
    blocks [q_heads, 64]` (int32 bit patterns of the u32 ids); `attend_blocks(blocks, b0, b1, include_recent) ->
    triples [q_heads * (2 + hd)]` laid out m | l | o; `attend_tokens(t0, t1) -> triples` for the dense cache;
    `merge(triples [world, q_heads * (2 + hd)]) -> out [heads*hd]` tensor."""
    score: Callable | None
    topk_pairs: Callable | None
    merge_pairs: Callable | None
    attend_blocks: Callable | None
    attend_tokens: Callable | None
    merge: Callable


def _all_gather(send: torch.Tensor, group=None) -> torch.Tensor:
    """One fixed-size message per rank, concatenated along a new leading dimension."""
    _, world = _world(group)
    recv = torch.empty((world * send.shape[0],) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
    dist.all_gather_into_tensor(recv, send.contiguous(), group=group)
    return recv.view((world,) + tuple(send.shape))


def compressed_split_k(legs: Legs, n_old_blocks: int, top_blocks: int, group=None):
    """One long sequence over the FP16-K / q4-V cache: score own blocks -> local top-k pairs -> all-gather pairs ->
    global top-k -> attend own selected blocks (the last rank adds the recent ring) -> all-gather triples -> merge.
    Every rank returns the full attention output and the block list (both as tensors of the legs' device)."""
    rank, world = _world(group)
    b0, b1 = block_ranges(n_old_blocks, world)[rank]
    pairs = legs.topk_pairs(legs.score(b0, b1), b0, top_blocks)
    blocks = legs.merge_pairs(_all_gather(pairs, group), top_blocks)
    triples = legs.attend_blocks(blocks, b0, b1, rank == world - 1)
    return legs.merge(_all_gather(triples, group)), blocks


def dense_split_k(legs: Legs, seq_len: int, group=None):
    """One long sequence over the dense FP16 cache: attend own token range -> all-gather triples -> merge."""
    rank, world = _world(group)
    t0, t1 = token_ranges(seq_len, world)[rank]
    return legs.merge(_all_gather(legs.attend_tokens(t0, t1), group))


def host_topk_pairs(scores: np.ndarray, index_base: int, top_blocks: int) -> np.ndarray:
    """Host statement of m40llm_topk_pairs_async (for plans and CPU tests): [q_heads, 64, 2] float32 whose [..., 1]
    holds the u32 block ids as raw bits."""
    scores = np.asarray(scores, np.float32)
    q_heads = scores.shape[0]
    sel = select_global_topk(scores, top_blocks) if scores.shape[1] else np.full((q_heads, MAX_TOP_BLOCKS), EMPTY_BLOCK, np.uint32)
    out = np.empty((q_heads, MAX_TOP_BLOCKS, 2), np.float32)
    ids = np.full((q_heads, MAX_TOP_BLOCKS), EMPTY_BLOCK, np.uint32)
    sc = np.full((q_heads, MAX_TOP_BLOCKS), np.float32(SCORE_FLOOR), np.float32)
    for h in range(q_heads):
        live = sel[h] != EMPTY_BLOCK
        ids[h, live] = sel[h, live] + np.uint32(index_base)
        sc[h, live] = scores[h, sel[h, live]]
    out[:, :, 0] = sc
    out[:, :, 1] = ids.view(np.float32)
    return out


def host_merge_pairs(pairs: np.ndarray, top_blocks: int) -> np.ndarray:
    """Host statement of m40llm_topk_merge_pairs_async: pairs [parts, q_heads, 64, 2] -> blocks [q_heads, 64] u32."""
    pairs = np.ascontiguousarray(pairs, np.float32)
    parts, q_heads = pairs.shape[0], pairs.shape[1]
    sc = pairs[..., 0].transpose(1, 0, 2).reshape(q_heads, parts * MAX_TOP_BLOCKS)
    ids = np.ascontiguousarray(pairs[..., 1]).view(np.uint32).transpose(1, 0, 2).reshape(q_heads, parts * MAX_TOP_BLOCKS)
    out = np.full((q_heads, MAX_TOP_BLOCKS), EMPTY_BLOCK, np.uint32)
    for h in range(q_heads):
        ok = np.flatnonzero(~np.isnan(sc[h]) & (sc[h] > np.float32(SCORE_FLOOR)) & (ids[h] != EMPTY_BLOCK))
        # descending score, ties to the lower block id
        order = ok[np.lexsort((ids[h][ok], -sc[h][ok]))][:top_blocks]
        out[h, :order.size] = ids[h][order]
    return out


class NativeLegs:
    """The legs over the CUDA library's split-K entry points. `lib` is the loaded C ABI (ctypes), `ctx`/`kv` its
    handles; `q` is a CUDA f32 tensor [q_heads * head_dim]. Every leg only enqueues: the kernels run on the context's
    decode stream, and `stream` (a torch view of that same stream, see `DeviceSplitK`) is where the collectives and
    the buffer allocations are ordered, so nothing here synchronises with the host."""

    def __init__(self, lib, ctx, kv, q: torch.Tensor, q_heads: int, head_dim: int, seq_id: int, seq_len: int):
        if not q.is_cuda:
            raise RuntimeError("NativeLegs needs CUDA tensors: the library has no CPU path")
        self.lib, self.ctx, self.kv, self.q = lib, ctx, kv, q.contiguous()
        self.qh, self.hd, self.seq, self.len = q_heads, head_dim, seq_id, seq_len
        self.dev = q.device
        # buffers are made once: a steady-state call allocates nothing
        z = lambda *s: torch.empty(s, dtype=torch.float32, device=self.dev)
        self._scores = None
        self._pairs = z(q_heads, MAX_TOP_BLOCKS, 2)
        self._blocks = torch.empty((q_heads, MAX_TOP_BLOCKS), dtype=torch.int32, device=self.dev)
        self._triples = z(q_heads * (2 + head_dim))
        self._out = z(q_heads * head_dim)

    def _p(self, t: torch.Tensor, offset_floats: int = 0):
        return C.c_void_p(t.data_ptr() + 4 * offset_floats)

    def _check(self, rc: int, what: str):
        if rc != 0:
            raise RuntimeError(f"{what} failed: {rc}")

    def score(self, b0: int, b1: int) -> torch.Tensor:
        n = b1 - b0
        if self._scores is None or self._scores.shape[1] != max(n, 1):
            self._scores = torch.empty((self.qh, max(n, 1)), dtype=torch.float32, device=self.dev)
        if n > 0:
            self._check(self.lib.m40llm_kvcache_score_old_blocks_async(self.ctx, self.kv, self.seq, self._p(self.q), self.qh,
                                                                       self.len, b0, b1, self._p(self._scores)),
                        "m40llm_kvcache_score_old_blocks_async")
        return self._scores[:, :n]

    def topk_pairs(self, scores: torch.Tensor, b0: int, top: int) -> torch.Tensor:
        n = scores.shape[1]
        self._check(self.lib.m40llm_topk_pairs_async(self.ctx, self._p(self._scores), self.qh, n, self._scores.shape[1], b0,
                                                     top, self._p(self._pairs)), "m40llm_topk_pairs_async")
        return self._pairs

    def merge_pairs(self, pairs: torch.Tensor, top: int) -> torch.Tensor:
        self._check(self.lib.m40llm_topk_merge_pairs_async(self.ctx, self._p(pairs), pairs.shape[0], self.qh, top,
                                                           self._p(self._blocks), None), "m40llm_topk_merge_pairs_async")
        return self._blocks

    def attend_blocks(self, blocks: torch.Tensor, b0: int, b1: int, include_recent: bool) -> torch.Tensor:
        t = self._triples
        self._check(self.lib.m40llm_attention_compressed_selected_partial_async(
            self.ctx, self.kv, self.seq, self._p(self.q), self.qh, self.len, self._p(blocks), b0, b1,
            1 if include_recent else 0, self._p(t), self._p(t, self.qh), self._p(t, 2 * self.qh)),
            "m40llm_attention_compressed_selected_partial_async")
        return t

    def attend_tokens(self, t0: int, t1: int) -> torch.Tensor:
        t = self._triples
        self._check(self.lib.m40llm_attention_last_token_f32_gqa_partial_async(
            self.ctx, self.kv, self.seq, self._p(self.q), self.qh, t0, t1, self._p(t), self._p(t, self.qh),
            self._p(t, 2 * self.qh)), "m40llm_attention_last_token_f32_gqa_partial_async")
        return t

    def merge(self, triples: torch.Tensor) -> torch.Tensor:
        self._check(self.lib.m40llm_attention_merge_gathered_async(self.ctx, self._p(triples), triples.shape[0], self.qh,
                                                                   self.hd, self._p(self._out)),
                    "m40llm_attention_merge_gathered_async")
        return self._out

    def legs(self) -> Legs:
        return Legs(self.score, self.topk_pairs, self.merge_pairs, self.attend_blocks, self.attend_tokens, self.merge)


class DeviceSplitK:
    """Split-K attention of one long sequence with everything enqueued on the library's decode stream: the stream is
    wrapped as a torch stream, made current around each call, and the NCCL all-gathers are ordered on it like the
    kernels. A call returns once the work is enqueued; synchronise the decode stream (or time with events on it)
    afterwards."""

    def __init__(self, lib, ctx, kv, q: torch.Tensor, q_heads: int, head_dim: int, seq_id: int, seq_len: int, group=None):
        handle = C.c_void_p()
        rc = lib.m40llm_context_stream_handle(ctx, 1, C.byref(handle))
        if rc != 0 or not handle.value:
            raise RuntimeError(f"m40llm_context_stream_handle failed: {rc}")
        self.stream = torch.cuda.ExternalStream(handle.value, device=q.device)
        self.group = group
        with torch.cuda.stream(self.stream):
            self.native = NativeLegs(lib, ctx, kv, q, q_heads, head_dim, seq_id, seq_len)
        self._legs = self.native.legs()

    def compressed(self, n_old_blocks: int, top_blocks: int):
        with torch.cuda.stream(self.stream):
            return compressed_split_k(self._legs, n_old_blocks, top_blocks, self.group)

    def dense(self, seq_len: int):
        with torch.cuda.stream(self.stream):
            return dense_split_k(self._legs, seq_len, self.group)

    def capture(self, fn):
        """Runs `fn()` once eagerly (scratch arenas and communicators exist afterwards), then captures a second run --
        library kernels and NCCL collectives alike, everything `fn` enqueues on the decode stream -- into a CUDA graph.
        Returns (replay, result): `replay()` enqueues the whole chain with one graph launch, `result` is what the
        captured run returned (tensors that every replay rewrites)."""
        with torch.cuda.stream(self.stream):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=self.stream, capture_error_mode="thread_local"):
            result = fn()

        def replay():
            with torch.cuda.stream(self.stream):
                graph.replay()

        self._graphs = getattr(self, "_graphs", []) + [graph]  # keep the graph (and its memory pool) alive
        return replay, result

    def capture_compressed(self, n_old_blocks: int, top_blocks: int):
        """One compressed split-K call captured as a CUDA graph: (replay, out, blocks). The eager call costs ~100 us of
        host enqueue time (five library calls, two collectives, their stream hand-overs); a replay costs what the device
        needs."""
        replay, (out, blocks) = self.capture(lambda: compressed_split_k(self._legs, n_old_blocks, top_blocks, self.group))
        return replay, out, blocks
