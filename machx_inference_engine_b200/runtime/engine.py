"""Serving engine: paged KV blocks with hash-based prefix sharing, a continuous-batching scheduler
with chunked prefill, the model runner (CUDA-graphed decode) and the public ``LLMEngine`` API.

What the reference does one request at a time behind a mutex (src/engine/engine.cpp:444-920:
encode -> budget check -> prefix-cache restore -> chunked prefill -> decode loop with a 4-byte
readback per token) is done here for many requests per step: every step is one model forward
over a ragged batch (prefill chunks and single decode tokens mixed), one batched sampler launch
and one device->host copy of the sampled ids.  The prefix cache keeps the reference's semantics
(longest cached token prefix is not recomputed; LRU eviction; src/core/prefix_cache.cpp:37-136)
but works at KV-block granularity so hits are shared between live requests without copies.
"""
from __future__ import annotations

import hashlib
import itertools
import time
from collections import OrderedDict, deque
from dataclasses import dataclass, field
from typing import Callable, Iterable, Optional

import torch

from .. import ops
from ..models.transformer import KV_BLOCK, ForwardBatch


@dataclass
class SamplingParams:
    """Reference parity: SamplingParams in include/ie/engine.hpp:43-76 (temperature 0 = greedy)."""
    temperature: float = 0.0
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    max_tokens: int = 128            # <= 0: until the context is full
    seed: int = 0
    stop_ids: tuple = ()
    ignore_eos: bool = False


class ContextLengthExceeded(ValueError):
    pass


class OutOfBlocks(RuntimeError):
    pass


@dataclass
class Sequence:
    seq_id: int
    prompt: list
    params: SamplingParams
    tokens: list = field(default_factory=list)         # prompt + generated
    n_computed: int = 0                                # tokens whose KV is in the cache
    blocks: list = field(default_factory=list)
    n_cached_prefix: int = 0
    finished: bool = False
    finish_reason: str = ""
    state_slot: int = -1
    restore_hash: Optional[bytes] = None       # hybrid models: block hash whose recurrent-state snapshot has to be restored into the slot
    restore_snap: Optional[object] = None      # ... and the snapshot itself, held from the prefix match until the restore (see Scheduler.schedule)
    h_last: Optional[torch.Tensor] = None      # hidden state of the last computed position (speculative decoding)
    t_arrival: float = 0.0
    t_first_token: float = 0.0
    on_token: Optional[Callable] = None
    block_hashes: list = field(default_factory=list)

    @property
    def n_generated(self) -> int:
        return len(self.tokens) - len(self.prompt)


class BlockManager:
    """Free list + content-hash index over full blocks (prefix sharing) with LRU reuse of cached blocks."""

    def __init__(self, num_blocks: int, enable_prefix_cache: bool = True):
        self.num_blocks = num_blocks
        self.free = deque(range(1, num_blocks))           # block 0 is the null block
        self.ref = [0] * num_blocks
        self.hash_of = [None] * num_blocks
        self.by_hash: dict = {}
        self.evictable: OrderedDict = OrderedDict()       # cached blocks with ref 0, LRU order
        self.enable_prefix_cache = enable_prefix_cache
        self.hits = 0
        self.queries = 0

    def n_free(self) -> int:
        return len(self.free) + len(self.evictable)

    def _take(self) -> int:
        if self.free:
            return self.free.popleft()
        if self.evictable:
            b, _ = self.evictable.popitem(last=False)
            h = self.hash_of[b]
            if h is not None and self.by_hash.get(h) == b:
                del self.by_hash[h]
            self.hash_of[b] = None
            return b
        raise OutOfBlocks("KV block pool exhausted")

    def allocate(self, n: int) -> list:
        if n > self.n_free():
            raise OutOfBlocks("KV block pool exhausted")
        out = []
        for _ in range(n):
            b = self._take()
            self.ref[b] = 1
            out.append(b)
        return out

    def release(self, blocks: Iterable[int]) -> None:
        for b in blocks:
            self.ref[b] -= 1
            if self.ref[b] == 0:
                if self.hash_of[b] is not None and self.enable_prefix_cache:
                    self.evictable[b] = True
                else:
                    self.hash_of[b] = None
                    self.free.append(b)

    @staticmethod
    def chain_hash(prev: Optional[bytes], tokens: list) -> bytes:
        h = hashlib.blake2b(digest_size=16)
        h.update(prev or b"root")
        h.update(b"".join(int(t).to_bytes(4, "little", signed=True) for t in tokens))
        return h.digest()

    def match_prefix(self, tokens: list) -> tuple[list, list]:
        """Longest run of cached full blocks for ``tokens`` -> (block ids with a reference taken, their hashes)."""
        self.queries += 1
        if not self.enable_prefix_cache:
            return [], []
        blocks, hashes, prev = [], [], None
        # never match the whole prompt: the last token must be recomputed to produce logits
        usable = (len(tokens) - 1) // KV_BLOCK
        for i in range(usable):
            h = self.chain_hash(prev, tokens[i * KV_BLOCK:(i + 1) * KV_BLOCK])
            b = self.by_hash.get(h)
            if b is None:
                break
            if self.ref[b] == 0:
                self.evictable.pop(b, None)
            self.ref[b] += 1
            blocks.append(b)
            hashes.append(h)
            prev = h
        if blocks:
            self.hits += 1
        return blocks, hashes

    def publish(self, seq: Sequence) -> None:
        """Register the sequence's newly completed full blocks in the hash index."""
        if not self.enable_prefix_cache:
            return
        n_full = seq.n_computed // KV_BLOCK
        while len(seq.block_hashes) < n_full:
            i = len(seq.block_hashes)
            prev = seq.block_hashes[-1] if seq.block_hashes else None
            h = self.chain_hash(prev, seq.tokens[i * KV_BLOCK:(i + 1) * KV_BLOCK])
            seq.block_hashes.append(h)
            b = seq.blocks[i]
            if h not in self.by_hash:
                self.by_hash[h] = b
                self.hash_of[b] = h


@dataclass
class EngineOptions:
    """Reference parity: EngineOptions in include/ie/engine.hpp (ctx, gpus, int8 kv, spec); new: batching knobs."""
    max_ctx: int = 8192
    max_batch_tokens: int = 8192        # token budget of one step (prefill chunk size)
    max_seqs: int = 64
    num_blocks: int = 0                 # 0: sized from max_seqs * max_ctx
    kv_memory_fraction: float = 0.0     # >0: size the pool from free device memory instead
    enable_prefix_cache: bool = True
    cuda_graphs: bool = True
    graph_batch_sizes: tuple = (1, 2, 4, 8, 16, 32, 64)
    eos_ids: tuple = ()
    spec_k: int = 0                     # MTP draft length (hybrid models with an MTP head)
    max_state_snapshots: int = 12       # hybrid models: recurrent-state snapshots kept for prefix reuse
    prefill_graphs: bool = True         # replay single-sequence prefill chunks of 512/1024/2048/4096/8192 tokens (or the full step budget) as CUDA graphs
    kv_dtype: str = "bf16"              # "int8": K/V rows stored as int8 with a per-row scale (halves the cache; `--int8-kv`)


class Scheduler:
    def __init__(self, opts: EngineOptions, bm: BlockManager, n_state_slots: int = 0, state_prefix: Optional[Callable] = None):
        self.opts, self.bm = opts, bm
        self.waiting: deque = deque()
        self.running: list = []
        self.free_state = deque(range(n_state_slots))
        self.uses_state = n_state_slots > 0
        self.state_prefix = state_prefix       # hashes -> number of leading blocks that end on a stored recurrent-state snapshot

    def add(self, seq: Sequence) -> None:
        self.waiting.append(seq)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _ensure_blocks(self, seq: Sequence, upto: int) -> bool:
        need = (upto + KV_BLOCK - 1) // KV_BLOCK - len(seq.blocks)
        if need <= 0:
            return True
        if need > self.bm.n_free():
            return False
        seq.blocks.extend(self.bm.allocate(need))
        return True

    def schedule(self) -> list:
        """Returns [(seq, n_new_tokens)]: every running sequence decodes one token, then waiting
        sequences get prefill chunks while the token budget lasts."""
        budget = self.opts.max_batch_tokens
        plan = []
        # decode first: latency of running requests is never starved by new prompts
        for seq in list(self.running):
            if seq.n_computed < len(seq.tokens) - 1:
                continue                                   # still prefilling: handled below
            if not self._ensure_blocks(seq, len(seq.tokens)):
                self._preempt(seq)
                continue
            plan.append((seq, 1))
            budget -= 1
        for seq in list(self.running):
            if seq.n_computed < len(seq.tokens) - 1 and budget > 0:
                n = min(budget, len(seq.tokens) - seq.n_computed)
                if self._ensure_blocks(seq, seq.n_computed + n):
                    plan.append((seq, n))
                    budget -= n
        while self.waiting and budget > 0 and len(self.running) < self.opts.max_seqs:
            seq = self.waiting[0]
            if self.uses_state and not self.free_state:
                break
            if not seq.blocks and seq.n_computed == 0:
                blocks, hashes = self.bm.match_prefix(seq.tokens)
                if self.uses_state:
                    # a recurrent model can resume only where its state was saved: keep the longest such prefix of the cached blocks
                    # The snapshot is held by the sequence from here on: admission can be deferred for any number of steps (no free
                    # blocks), and in the meantime other sequences may push it out of the LRU snapshot cache.  Resuming at the cached
                    # position without it would continue on the slot's previous occupant's state.
                    keep, snap = self.state_prefix(hashes) if (self.state_prefix and hashes) else (0, None)
                    self.bm.release(blocks[keep:])
                    blocks, hashes = blocks[:keep], hashes[:keep]
                    seq.restore_hash = hashes[-1] if keep else None
                    seq.restore_snap = snap if keep else None
                seq.blocks, seq.block_hashes = blocks, hashes
                seq.n_computed = seq.n_cached_prefix = len(blocks) * KV_BLOCK
            n = min(budget, len(seq.tokens) - seq.n_computed)
            if not self._ensure_blocks(seq, seq.n_computed + n):
                break
            self.waiting.popleft()
            if self.uses_state:
                seq.state_slot = self.free_state.popleft()
            self.running.append(seq)
            plan.append((seq, n))
            budget -= n
        return plan

    def _preempt(self, seq: Sequence) -> None:
        """Out of blocks: push the sequence back to the queue; its KV is recomputed later."""
        self.running.remove(seq)
        self.bm.release(seq.blocks)
        seq.blocks, seq.block_hashes, seq.n_computed = [], [], 0
        seq.restore_hash = seq.restore_snap = None
        if seq.state_slot >= 0:
            self.free_state.append(seq.state_slot)
            seq.state_slot = -1
        self.waiting.appendleft(seq)

    def finish(self, seq: Sequence) -> None:
        if seq in self.running:
            self.running.remove(seq)
        self.bm.release(seq.blocks)
        seq.blocks = []
        if seq.state_slot >= 0:
            self.free_state.append(seq.state_slot)
            seq.state_slot = -1


class LLMEngine:
    """Public API: ``add_request`` / ``step`` for servers, ``generate`` for batch use."""

    def __init__(self, model, opts: Optional[EngineOptions] = None):
        self.model = model
        self.opts = opts or EngineOptions()
        self.device = model.device
        cfg = model.cfg
        o = self.opts
        blocks_per_seq = (o.max_ctx + KV_BLOCK - 1) // KV_BLOCK
        nb = o.num_blocks or (o.max_seqs * blocks_per_seq + 1)
        if o.kv_memory_fraction > 0 and self.device.type == "cuda":
            free, _ = torch.cuda.mem_get_info(self.device)
            from ..models.transformer import KVCache
            per = max(1, KVCache.bytes_per_block(len(model.attn_layers), model.n_kv_local, cfg.head_dim, o.kv_dtype))
            nb = max(blocks_per_seq + 1, int(free * o.kv_memory_fraction) // per)
        self.max_blocks_per_seq = blocks_per_seq
        self.kv = model.new_kv_cache(nb, o.kv_dtype) if o.kv_dtype != "bf16" else model.new_kv_cache(nb)
        n_state = o.max_seqs if getattr(model, "needs_state", False) else 0
        self.state = model.new_state(n_state + 1) if n_state else None      # the extra slot absorbs graph-padding rows
        self.bm = BlockManager(nb, o.enable_prefix_cache)
        # recurrent-state snapshots at block boundaries, keyed by the chained block hash, LRU (the reference keeps KV slab +
        # DeltaNet snapshot per trie endpoint: include/ie/prefix_cache.hpp:39-118, fleet_prefix_cache.hpp:36-98; max 12 entries)
        self.state_cache: OrderedDict = OrderedDict()
        self.sched = Scheduler(o, self.bm, n_state, state_prefix=self._state_prefix if n_state else None)
        self._ids = itertools.count()
        self._graphs: dict = {}
        self._graph_pool = None
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "graph_replays": 0, "h2d_bytes": 0, "d2h_bytes": 0,
                      "spec_rounds": 0, "spec_drafted": 0, "spec_accepted": 0}
        self.eos_ids = set(o.eos_ids)
        # self-speculative decoding needs a draft head; models with recurrent state also need their state pool (for the rollback)
        self.spec_k = o.spec_k if (o.spec_k > 0 and getattr(model, "mtp", None) is not None
                                   and (self.state is not None or not getattr(model, "needs_state", False))) else 0

    # ------------------------------------------------------------------ recurrent-state prefix snapshots (hybrid models)
    def _state_prefix(self, hashes: list):
        """(number of leading blocks that end on a stored snapshot, that snapshot)."""
        for n in range(len(hashes), 0, -1):
            snap = self.state_cache.get(hashes[n - 1])
            if snap is not None:
                self.state_cache.move_to_end(hashes[n - 1])
                return n, snap
        return 0, None

    def _restore_states(self, plan: list) -> None:
        for seq, _ in plan:
            if seq.restore_hash is not None:
                snap = seq.restore_snap if seq.restore_snap is not None else self.state_cache.get(seq.restore_hash)
                if snap is None:          # cannot happen while the sequence holds its snapshot; never resume on a foreign state
                    raise RuntimeError("recurrent-state snapshot of a matched prefix is gone")
                self.state.restore(seq.state_slot, snap)
                seq.restore_hash = seq.restore_snap = None

    def _save_states(self, plan: list) -> None:
        if self.state is None or not self.opts.enable_prefix_cache:
            return
        for seq, n in plan:
            if n > 1 and seq.n_computed % KV_BLOCK == 0 and seq.n_computed <= len(seq.prompt) and len(seq.block_hashes) >= seq.n_computed // KV_BLOCK > 0:
                key = seq.block_hashes[seq.n_computed // KV_BLOCK - 1]
                if key not in self.state_cache:
                    self.state_cache[key] = self.state.snapshot(seq.state_slot)
                    while len(self.state_cache) > self.opts.max_state_snapshots:
                        self.state_cache.popitem(last=False)

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_ids: list, params: Optional[SamplingParams] = None, on_token: Optional[Callable] = None) -> Sequence:
        params = params or SamplingParams()
        if len(prompt_ids) == 0:
            raise ValueError("empty prompt")
        if len(prompt_ids) >= self.opts.max_ctx - 8:       # the reference's budget guard (engine.cpp:452-463)
            raise ContextLengthExceeded(f"prompt of {len(prompt_ids)} tokens does not fit the context of {self.opts.max_ctx}")
        seq = Sequence(next(self._ids), list(prompt_ids), params, tokens=list(prompt_ids), t_arrival=time.perf_counter(), on_token=on_token)
        self.sched.add(seq)
        return seq

    def abort(self, seq: Sequence) -> None:
        if seq in self.sched.waiting:
            self.sched.waiting.remove(seq)
        if not seq.finished:
            seq.finished, seq.finish_reason = True, "abort"
            self.sched.finish(seq)

    def has_work(self) -> bool:
        return self.sched.has_work()

    # ------------------------------------------------------------------ one step
    def step(self) -> list:
        """Runs one forward over the scheduled batch; returns [(seq, token, finished)] for sequences that produced a token."""
        plan = self.sched.schedule()
        if not plan:
            if self.sched.waiting and not self.sched.running:
                raise OutOfBlocks("a waiting request cannot be scheduled: KV pool too small for its prompt")
            return []
        sampled_rows = [i for i, (s, n) in enumerate(plan) if s.n_computed + n == len(s.tokens)]
        if self.spec_k and len(plan) == 1 and plan[0][1] == 1 and sampled_rows and self._spec_ok(plan[0][0]):
            done = self._spec_step(plan[0][0])
            if done is not None:
                return done
        tokens = self._run(plan, sampled_rows)
        out = []
        for (seq, n) in plan:
            seq.n_computed += n
        for row, i in enumerate(sampled_rows):
            seq, n = plan[i]
            tok = int(tokens[row])
            if not 0 <= tok < self.model.cfg.vocab:       # never hand an id outside the vocabulary to the history / detokeniser / callbacks
                seq.finished, seq.finish_reason = True, "error"
                out.append((seq, -1, True))
                continue
            if seq.n_generated == 0:
                seq.t_first_token = time.perf_counter()
            seq.tokens.append(tok)
            self._check_finish(seq, tok)
            if seq.on_token is not None:
                seq.on_token(seq, tok)
            out.append((seq, tok, seq.finished))
        for seq, n in plan:
            if n > 1:
                self.stats["prefill_tokens"] += n
            else:
                self.stats["decode_tokens"] += 1
            self.bm.publish(seq)
        self._save_states(plan)
        for seq, n in plan:
            if seq.finished:
                self.sched.finish(seq)
        self.stats["steps"] += 1
        return out

    def _check_finish(self, seq: Sequence, tok: int) -> None:
        p = seq.params
        if not p.ignore_eos and (tok in self.eos_ids or tok in p.stop_ids):
            seq.finished, seq.finish_reason = True, "stop"
        elif p.max_tokens > 0 and seq.n_generated >= p.max_tokens:
            seq.finished, seq.finish_reason = True, "length"
        elif len(seq.tokens) >= self.opts.max_ctx:
            seq.finished, seq.finish_reason = True, "length"

    # ------------------------------------------------------------------ batch assembly + execution
    def _build_batch(self, plan: list, sampled_rows: list, pad_to: int = 0):
        ids, pos, slots, cu, lens, tables, logit_rows = [], [], [], [0], [], [], []
        for i, (seq, n) in enumerate(plan):
            s0 = seq.n_computed
            ids.extend(seq.tokens[s0:s0 + n])
            pos.extend(range(s0, s0 + n))
            for p_ in range(s0, s0 + n):
                slots.append(seq.blocks[p_ // KV_BLOCK] * KV_BLOCK + p_ % KV_BLOCK)
            cu.append(cu[-1] + n)
            lens.append(s0 + n)
            tables.append(seq.blocks)
        for i in sampled_rows:
            logit_rows.append(cu[i + 1] - 1)
        B = len(plan)
        for _ in range(max(0, pad_to - B)):                # graph padding: null sequences of one token in block 0
            ids.append(0); pos.append(0); slots.append(-1); cu.append(cu[-1] + 1); lens.append(1); tables.append([0])
            logit_rows.append(cu[-1] - 1)
        mb = self.max_blocks_per_seq
        bt = torch.zeros(len(tables), mb, dtype=torch.int32)
        for r, t in enumerate(tables):
            if len(t) > mb:
                raise ContextLengthExceeded("sequence outgrew the block table")
            bt[r, :len(t)] = torch.tensor(t, dtype=torch.int32)
        extra = {}
        if self.state is not None:
            pad_slot = self.state.n_slots - 1
            extra["state_slots"] = torch.tensor([s.state_slot for s, _ in plan] + [pad_slot] * max(0, pad_to - B), dtype=torch.int32)
        host = {
            **extra,
            "ids": torch.tensor(ids, dtype=torch.int32), "positions": torch.tensor(pos, dtype=torch.int32),
            "slot_map": torch.tensor(slots, dtype=torch.int64), "block_table": bt, "seq_lens": torch.tensor(lens, dtype=torch.int32),
            "cu_q": torch.tensor(cu, dtype=torch.int32), "logit_rows": torch.tensor(logit_rows, dtype=torch.int64),
        }
        return host, max(n for _, n in plan)

    def _to_device(self, host: dict) -> dict:
        dev = {}
        for k, v in host.items():
            if self.device.type == "cuda":
                v = v.pin_memory()
            dev[k] = v.to(self.device, non_blocking=True)
            self.stats["h2d_bytes"] += v.numel() * v.element_size()
        return dev

    def _sampling_tensors(self, seqs: list, pad_to: int = 0):
        n = max(len(seqs), pad_to)
        t = torch.zeros(n); k = torch.zeros(n, dtype=torch.int32); p = torch.ones(n); m = torch.zeros(n)
        for i, s in enumerate(seqs):
            t[i], k[i], p[i], m[i] = s.params.temperature, s.params.top_k, s.params.top_p, s.params.min_p
        return t, k, p, m

    def _run(self, plan: list, sampled_rows: list) -> list:
        if self.state is not None:
            self._restore_states(plan)
        decode_only = all(n == 1 for _, n in plan) and len(sampled_rows) == len(plan)
        seqs = [plan[i][0] for i in sampled_rows]
        greedy = all(s.params.temperature <= 0 and s.params.repetition_penalty == 1.0 for s in seqs)
        par = getattr(self.model, "par", None)
        # graphs hold only this library's kernels: the NCCL baseline path (no fused collectives) and the layer split (NCCL
        # point-to-point hand-offs between the stages) run eagerly
        nccl_path = par is not None and par.enabled and (par.fused is None or par.mode == "pp")
        use_graph = (decode_only and greedy and self.opts.cuda_graphs and self.device.type == "cuda"
                     and (self.state is None or all(s.n_computed > 0 for s, _ in plan))
                     and len(plan) <= max(self.opts.graph_batch_sizes) and not nccl_path and not self.spec_k)
        if use_graph:
            return self._run_graph(plan)
        if (self.opts.cuda_graphs and self.opts.prefill_graphs and self.opts.kv_dtype == "bf16" and self.device.type == "cuda" and not nccl_path
                and len(plan) == 1
                and (plan[0][1] in (512, 1024, 2048, 4096, 8192) or (plan[0][1] == self.opts.max_batch_tokens and plan[0][1] % KV_BLOCK == 0
                                                                      and plan[0][1] >= 256)) and not self.spec_k):
            return self._run_prefill_graph(plan, sampled_rows, seqs)
        host, max_q = self._build_batch(plan, sampled_rows)
        dev = self._to_device(host)
        fb = ForwardBatch(dev["ids"], dev["positions"], dev["slot_map"], dev["block_table"], dev["seq_lens"], dev["cu_q"], max_q,
                          logit_rows=dev["logit_rows"] if sampled_rows else dev["cu_q"][1:2].long() - 1)
        fb.max_kv_len = max(s.n_computed + n for s, n in plan)
        if self.state is not None:
            fb.state_slots_host = [s.state_slot for s, _ in plan]
            fb.state_slots = dev["state_slots"]
            fb.q_lens_host = [n for _, n in plan]
            fb.start_host = [s.n_computed for s, _ in plan]
        fb.want_hidden = bool(self.spec_k) and bool(sampled_rows)
        logits = self.model.forward(fb, self.kv, self.state) if self.state is not None else self.model.forward(fb, self.kv)
        if fb.want_hidden:
            logits, hidden = logits
            for r, s in enumerate(seqs):
                s.h_last = hidden[r:r + 1]
        if not sampled_rows:
            return []
        toks = self._sample(logits, seqs)
        out = toks.cpu()
        self.stats["d2h_bytes"] += out.numel() * 4
        return out.tolist()

    def _sample(self, logits: torch.Tensor, seqs: list) -> torch.Tensor:
        if all(s.params.temperature <= 0 and s.params.repetition_penalty == 1.0 for s in seqs):
            return ops.argmax(logits)
        dev = logits.device
        if any(s.params.repetition_penalty != 1.0 for s in seqs):
            uniq = [sorted(set(s.tokens)) for s in seqs]
            width = max(len(u) for u in uniq)
            ids = torch.full((len(seqs), width), -1, dtype=torch.int32)
            for i, u in enumerate(uniq):
                ids[i, :len(u)] = torch.tensor(u, dtype=torch.int32)
            pen = torch.tensor([s.params.repetition_penalty for s in seqs], dtype=torch.float32)
            ops.rep_penalty(logits, ids.to(dev), pen.to(dev))
        t, k, p, m = self._sampling_tensors(seqs)
        rng = torch.tensor([_seed_state(s.params.seed, s.seq_id, s.n_generated) for s in seqs], dtype=torch.int64)
        return ops.sample(logits, t.to(dev), k.to(dev), p.to(dev), m.to(dev), rng.to(dev))

    # ------------------------------------------------------------------ MTP self-speculative decode (greedy, lossless)
    def _spec_ok(self, seq: Sequence) -> bool:
        p = seq.params
        return (p.temperature <= 0 and p.repetition_penalty == 1.0 and getattr(seq, "h_last", None) is not None
                and len(seq.tokens) + self.spec_k + 1 < self.opts.max_ctx)

    def _spec_step(self, seq: Sequence):
        """One draft-verify round (src/model/qwen35_dense.cpp:1168-1264): the MTP head drafts K tokens after the pending
        token, ONE target forward over [pending, drafts] in checkpoint mode verifies them, the longest agreeing prefix plus
        the target's own next token are committed, and the recurrent state is rolled back to the last accepted position."""
        K = self.spec_k
        p0 = seq.n_computed
        if not self.sched._ensure_blocks(seq, p0 + K + 1):
            return None
        # (a head that reads the target's cache -- Gemma-4's assistant -- takes the sequence's pages and position; others ignore it)
        ctx = {"kv": self.kv, "pos": p0, "block_table": torch.tensor([seq.blocks], dtype=torch.int32, device=self.device)}
        drafts = self.model.mtp.draft(seq.h_last, seq.tokens[-1], K, ctx)
        base = list(seq.tokens)
        seq.tokens = base + drafts
        try:
            host, max_q = self._build_batch([(seq, K + 1)], [])
        finally:
            seq.tokens = base
        host["logit_rows"] = torch.arange(K + 1, dtype=torch.int64)
        dev = self._to_device(host)
        fb = ForwardBatch(dev["ids"], dev["positions"], dev["slot_map"], dev["block_table"], dev["seq_lens"], dev["cu_q"], max_q,
                          logit_rows=dev["logit_rows"], want_hidden=True)
        fb.q_lens_host, fb.start_host = [K + 1], [p0]
        if self.state is not None:
            fb.state_slots_host = [seq.state_slot]
            fb.state_slots = dev["state_slots"]
            logits, hidden = self.model.forward(fb, self.kv, self.state, checkpoint=True)
        else:
            # no recurrent state: rejected drafts leave stale keys behind the committed position, and the next forward overwrites them
            logits, hidden = self.model.forward(fb, self.kv, None)
        targ = ops.argmax(logits).cpu().tolist()
        self.stats["d2h_bytes"] += 4 * (K + 1)
        n = 0
        while n < K and drafts[n] == targ[n]:
            n += 1
        accepted = n + 1                       # verified input rows kept: the pending token and n drafts
        if accepted < K + 1 and self.state is not None:
            self.state.commit(seq.state_slot, accepted - 1)
        seq.h_last = hidden[accepted - 1:accepted].clone()
        seq.n_computed = p0 + accepted
        self.stats["spec_rounds"] += 1
        self.stats["spec_drafted"] += K
        self.stats["spec_accepted"] += n
        out = []
        for tok in drafts[:n] + [targ[n]]:
            if seq.n_generated == 0:
                seq.t_first_token = time.perf_counter()
            seq.tokens.append(tok)
            self._check_finish(seq, tok)
            if seq.on_token is not None:
                seq.on_token(seq, tok)
            out.append((seq, tok, seq.finished))
            self.stats["decode_tokens"] += 1
            if seq.finished:
                break
        if seq.finished:
            self.sched.finish(seq)
        self.stats["steps"] += 1
        return out

    # ------------------------------------------------------------------ CUDA-graphed greedy decode
    def _run_graph(self, plan: list) -> list:
        B = len(plan)
        gb = next(b for b in self.opts.graph_batch_sizes if b >= B)
        host, _ = self._build_batch(plan, list(range(B)), pad_to=gb)
        g = self._graphs.get(gb)
        if g is None:
            g = self._capture(gb, host)
            self._graphs[gb] = g
        for k, v in host.items():
            g["in"][k].copy_(v.pin_memory(), non_blocking=True)
            self.stats["h2d_bytes"] += v.numel() * v.element_size()
        g["graph"].replay()
        from ..ops import cuda as kernels
        kernels._count(g["kernels"])
        self.stats["graph_replays"] += 1
        out = g["out"].cpu()
        self.stats["d2h_bytes"] += out.numel() * 4
        return out[:B].tolist()

    # ------------------------------------------------------------------ CUDA-graphed prefill chunks
    def _run_prefill_graph(self, plan: list, sampled_rows: list, seqs: list) -> list:
        """A single-sequence prefill chunk of n tokens (n a multiple of the KV block) has fixed shapes: its whole forward is one
        graph replay.  With tensor parallelism the per-kernel GPU time shrinks with the rank count while the host cost of
        ~500 launches does not, so an eager prefill becomes launch-bound; the graph removes that floor."""
        seq, n = plan[0]
        host, max_q = self._build_batch(plan, [0])            # always one logit row: the chunk's last token
        key = ("prefill", n)
        g = self._graphs.get(key)
        if self.state is not None and seq.n_computed == 0:
            self.state.reset([seq.state_slot])
        if g is None:
            g = self._capture(n, host, prefill_tokens=n)
            self._graphs[key] = g
        for k, v in host.items():
            g["in"][k].copy_(v.pin_memory(), non_blocking=True)
            self.stats["h2d_bytes"] += v.numel() * v.element_size()
        g["graph"].replay()
        from ..ops import cuda as kernels
        kernels._count(g["kernels"])
        self.stats["graph_replays"] += 1
        if not sampled_rows:
            return []
        toks = self._sample(g["logits"], seqs).cpu()
        self.stats["d2h_bytes"] += toks.numel() * 4
        return toks.tolist()

    def _capture(self, gb: int, host: dict, prefill_tokens: int = 0) -> dict:
        dev = {k: v.to(self.device) for k, v in host.items()}
        fb = ForwardBatch(dev["ids"], dev["positions"], dev["slot_map"], dev["block_table"], dev["seq_lens"], dev["cu_q"], prefill_tokens or 1,
                          logit_rows=dev["logit_rows"], state_slots=dev.get("state_slots"))
        fwd = (lambda: self.model.forward(fb, self.kv, self.state)) if self.state is not None else (lambda: self.model.forward(fb, self.kv))
        if prefill_tokens:
            return self._capture_with(fwd, dev, host, argmax=False)
        return self._capture_with(fwd, dev, host, argmax=True)

    def _capture_with(self, fwd, dev: dict, host: dict, argmax: bool) -> dict:
        post = ops.argmax if argmax else (lambda t: t)
        snap = None
        if self.state is not None:
            # the warm-up and capture forwards advance the recurrent state of the slots in this batch: put it back afterwards
            slots = sorted(set(host["state_slots"].tolist()))
            snap = {sl: self.state.snapshot(sl) for sl in slots}
        # warm up on a side stream (allocator, lazy kernel attributes), then capture
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            for _ in range(2):
                post(fwd())
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        from ..ops import cuda as kernels
        n0 = kernels.launches()
        with torch.cuda.graph(graph, pool=self._graph_pool):
            out = post(fwd())
        n_kernels = kernels.launches() - n0          # kernels recorded in the graph: every replay launches them again
        if snap is not None:
            for sl, sn in snap.items():
                self.state.restore(sl, sn)
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        return {"graph": graph, "in": dev, "out": out, "logits": out, "kernels": n_kernels}

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts: list, params: Optional[SamplingParams] = None) -> list:
        """Runs the prompts (lists of token ids) to completion; returns the generated ids per prompt."""
        seqs = [self.add_request(p, params) for p in prompts]
        while any(not s.finished for s in seqs):
            self.step()
        return [s.tokens[len(s.prompt):] for s in seqs]


def _seed_state(seed: int, seq_id: int, step: int) -> int:
    x = (seed * 0x9E3779B97F4A7C15 + seq_id * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB + 0x2545F4914F6CDD1D) & ((1 << 64) - 1)
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & ((1 << 64) - 1)
    x ^= x >> 27
    x = x or 1
    return x if x < (1 << 63) else x - (1 << 64)
