"""In-flight batching runtime for models defined as a ``layers.LayerStackModel``.

One ``InflightSession.step`` runs an arbitrary mix of sequences — a portion of one prompt of any length beside single
generated tokens of others — as one ragged batch over the model's kernels.  Between steps a sequence lives in

  * pages of the cache pools (one pool per caching layer and pass of a looped block — latent entries or keys and values —
    the same block ids in every pool), dealt by ``runtime.KVCacheManager`` (``reserve`` / ``release``), and
  * one slot of the state buffers (per layer that has them: the recurrence state and / or the carried inputs of its short
    convolutions), dealt by ``StateSlotManager``.

``InflightScheduler`` + ``InflightSession.generate`` are the generation entry point: admission by free slots and pages,
chunked prefill under a per-step token budget beside the running decodes, sampling with the library's sampling kernels
(``SamplingConfig``), release at end-of-sequence.  The reference's batch manager is closed source
(T/cpp/tensorrt_llm/batch_manager, a static library); its Python loop (T/tensorrt_llm/runtime/generation.py:782-997)
steps a fixed batch, which ``runtime.GenerationSession`` mirrors for LLaMA engines.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import torch

from . import ops
from .runtime import GenerationSequence, KVCacheManager, SamplingConfig


class StateSlotManager:
    """Fixed number of recurrent-state slots; a slot is handed on as it is (the kernels start a sequence that stands
    at position 0 from zeros whatever the slot holds)."""

    def __init__(self, slots: int):
        self.slots = slots
        self.free = list(range(slots))

    def acquire(self) -> int:
        if not self.free:
            raise RuntimeError("no free state slot")
        return self.free.pop(0)

    def release(self, slot: int):
        self.free.append(slot)


class RaggedBatch:
    """Device-side description of one step (see include/trtllm_b200_ragged.h), uploaded as ONE int32 buffer."""

    def __init__(self, entries, want_rows, device, max_blocks=None):
        """entries: [(token ids, past length, state slot, block ids[, the token before these, -1 for none])]; want_rows: row
        indices whose logits are wanted.  ``max_blocks`` pads the block table's row length (a replayed step graph needs it fixed)."""
        self.device = device
        self.max_blocks = max(1, max(len(e[3]) for e in entries), max_blocks or 0)
        host = self._pack(entries, want_rows)
        if torch.device(device).type == "cuda":
            host = host.pin_memory()
        self._host, self._dev = host, host.to(device, non_blocking=True)
        self._views()

    def _pack(self, entries, want_rows):
        tok_ids, tok_seq, tok_pos, tok_prev, start, length, past, slot, table = [], [], [], [], [], [], [], [], []
        for i, entry in enumerate(entries):
            toks, p, s, blocks = entry[:4]
            toks = list(toks)
            before = int(entry[4]) if len(entry) > 4 and entry[4] is not None else -1
            tok_prev += [before if p > 0 else -1] + toks[:-1]
            start.append(len(tok_ids))
            length.append(len(toks))
            past.append(p)
            slot.append(s)
            tok_ids += list(toks)
            tok_seq += [i] * len(toks)
            tok_pos += range(p, p + len(toks))
            table += list(blocks) + [-1] * (self.max_blocks - len(blocks))
        self.num_rows, self.num_seqs, self.num_want = len(tok_ids), len(entries), len(want_rows)
        self.max_len = max(length)        # host-side hints for kernels that size their grids by the longest portion
        self.max_pos = max(tok_pos)       # ... and by context length
        self._sizes = [len(tok_ids)] * 4 + [len(entries)] * 4 + [len(table), len(want_rows)]
        return torch.tensor(tok_ids + tok_seq + tok_pos + tok_prev + start + length + past + slot + table + list(want_rows),
                            dtype=torch.int32)

    def _views(self):
        off, views = 0, []
        for n in self._sizes:
            views.append(self._dev[off:off + n])
            off += n
        # tok_prev: the token before each row in its sequence (-1 at position 0) — part of a sequence's state between steps
        (self.tok_ids, self.tok_seq, self.tok_pos, self.tok_prev, self.seq_start, self.seq_len, self.seq_past, self.seq_slot,
         self.block_table, self.want_rows) = views

    def refill(self, entries, want_rows):
        """Same shape, new contents, SAME device addresses (the batch a captured step graph reads)."""
        sizes = self._sizes
        host = self._pack(entries, want_rows)
        if self._sizes != sizes:
            raise ValueError("refill() needs a batch of the same shape")
        self._host = host.pin_memory() if torch.device(self.device).type == "cuda" else host
        self._dev.copy_(self._host, non_blocking=True)


class StepContext:
    """What the layers see during one step."""

    def __init__(self, batch, pools, states, page):
        self.batch, self.pools, self.states, self.page = batch, pools, states, page
        self._tables = {}

    def rope_table(self, dims, base, scaling=None):
        """One table per (dims, base, frequency scaling) and step, shared by every layer that rotates that way."""
        key = (int(dims), float(base), tuple(scaling) if scaling else None)
        if key not in self._tables:
            self._tables[key] = ops.rope_table(self.batch.tok_pos, dims, base, scaling)
        return self._tables[key]


@dataclass
class _Live:
    handle: GenerationSequence
    slot: int
    length: int = 0
    last_token: int = -1               # the newest token it holds (models whose embedding reads the previous token)


class InflightSession:
    """Serves one ``LayerStackModel``.  ``max_tokens`` sizes the latent-cache pools (positions held by all live
    sequences together, each rounded up to whole pages); ``max_seqs`` is the number of state slots."""

    def __init__(self, model, max_tokens: int, max_seqs: int = 4, tokens_per_block: int = 64, device="cuda",
                 use_cuda_graph: bool = True):
        self.model, self.device, self.page = model, torch.device(device), int(tokens_per_block)
        self.use_cuda_graph = bool(use_cuda_graph) and self.device.type == "cuda"
        self._graphs = {}
        blocks = max(1, -(-int(max_tokens) // self.page))
        self.kv_cache_manager = KVCacheManager(blocks=blocks, tokens_per_block=self.page, max_blocks_per_seq=blocks)
        self.slot_manager = StateSlotManager(max_seqs)
        # keyed by (layer, pass): a layer that a looped block runs several times holds one pool / state per pass
        self.pools = {k: torch.empty((blocks * self.page, width), dtype=model.dtype, device=self.device)
                      for k, width in model.cache_layers().items()}
        self.states = {k: (torch.zeros((max_seqs, max(taps - 1, 1), ch), dtype=torch.float32, device=self.device),
                           torch.zeros((max_seqs, rec), dtype=torch.float32, device=self.device) if rec else None)
                       for k, (taps, ch, rec) in model.state_layers().items()}
        self.live = {}
        self._next_idx = 0

    # -- sequences ---------------------------------------------------------------------------------------------
    def _admit(self, seq_id):
        slot = self.slot_manager.acquire()
        self.live[seq_id] = _Live(GenerationSequence(seq_idx=self._next_idx, batch_idx=slot), slot)
        self._next_idx += 1
        return self.live[seq_id]

    def end(self, seq_id):
        """The sequence is finished: its pages and its state slot are free for the next one."""
        s = self.live.pop(seq_id)
        if s.handle in self.kv_cache_manager.allocated:
            self.kv_cache_manager.release(s.handle)
        self.slot_manager.release(s.slot)

    def length(self, seq_id) -> int:
        return self.live[seq_id].length

    # -- the step function -----------------------------------------------------------------------------------------
    def step(self, entries, on_layer=None):
        """entries: [(seq_id, new token ids, want)] — ``want`` lists the places among the new tokens whose logits are
        asked for.  A sequence is admitted at its first entry.  Returns fp32 logits [sum(len(want)), vocab] on the
        device (None when nothing is wanted), rows in the order of the entries and of ``want``."""
        rows, want_rows, n = [], [], 0
        fresh = []
        try:
            for seq_id, tokens, want in entries:
                if not len(tokens):
                    raise ValueError(f"sequence {seq_id!r} brings no token")
                s = self.live.get(seq_id)
                if s is None:
                    s = self._admit(seq_id)
                    fresh.append(seq_id)
                self.kv_cache_manager.reserve(s.handle, s.length + len(tokens))
                rows.append((tokens, s.length, s.slot, self.kv_cache_manager.blocks_of(s.handle), s.last_token))
                want_rows += [n + int(w) for w in want]
                n += len(tokens)
        except Exception:
            for seq_id in fresh:          # nothing ran: a step that cannot be placed leaves no half-admitted sequence
                self.end(seq_id)
            raise
        if (self.use_cuda_graph and on_layer is None and len(want_rows) == n
                and all(len(r[0]) == 1 for r in rows)):
            logits = self._generation_step_graph(rows)
        else:
            batch = RaggedBatch(rows, want_rows, self.device)
            ctx = StepContext(batch, self.pools, self.states, self.page)
            x = self.model.forward(ctx, on_layer=on_layer)
            self.last_batch = batch       # keeps the pinned upload buffer alive until the next step
            logits = self.model.logits(x, batch.want_rows) if want_rows else None
        for seq_id, tokens, _ in entries:
            self.live[seq_id].length += len(tokens)
            self.live[seq_id].last_token = int(tokens[-1])
        return logits

    def _generation_step_graph(self, rows):
        """A step in which every sequence brings ONE token and wants its logits (a generation step) is launch-bound:
        ~20 kernels per layer against a few hundred microseconds of work.  Such steps are captured once per (number of
        sequences, block-table width) as a CUDA graph over a batch description at fixed device addresses and replayed
        with new contents; everything else of the step (positions, pages, slots) is data the kernels read."""
        B = len(rows)
        width = -(-max(len(r[3]) for r in rows) // 8) * 8
        key = (B, width)
        want = list(range(B))
        g = self._graphs.get(key)
        if g is None:
            batch = RaggedBatch(rows, want, self.device, max_blocks=width)
            batch.max_pos = width * self.page - 1            # sizes the key split for every length this table holds
            ctx = StepContext(batch, self.pools, self.states, self.page)
            logits = self.model.logits(self.model.forward(ctx), batch.want_rows)      # this step, eagerly
            out = logits.clone()
            graph, captured = torch.cuda.CUDAGraph(), None
            try:
                with torch.cuda.graph(graph):             # records, does not run: states and caches are not touched
                    cctx = StepContext(batch, self.pools, self.states, self.page)
                    captured = self.model.logits(self.model.forward(cctx), batch.want_rows)
            except RuntimeError:
                self.use_cuda_graph = False                   # capture not possible here: stay with eager launches
                return out
            if len(self._graphs) >= 32:
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[key] = (graph, batch, captured)
            return out
        graph, batch, captured = g
        batch.refill(rows, want)
        batch.max_pos = width * self.page - 1
        graph.replay()
        return captured.clone()

    # -- generation ------------------------------------------------------------------------------------------------
    def generate(self, prompts, max_new_tokens: int, sampling_config: SamplingConfig = None, max_step_tokens: int = 512):
        """Greedy / sampled generation of ``max_new_tokens`` per prompt through the scheduler.  ``prompts``: lists of
        token ids (any number; they queue for slots and pages).  Returns one list of new ids per prompt; a sequence
        stops early at ``sampling_config.end_id`` (kept as its last id)."""
        sc = sampling_config or SamplingConfig(end_id=None)
        if sc.num_beams != 1 or sc.repetition_penalty != 1.0 or sc.min_length > 1:
            raise NotImplementedError("in-flight generation: beam width 1, no repetition penalty / min_length")
        sched = InflightScheduler(self, max_step_tokens)
        for i, p in enumerate(prompts):
            sched.add(("gen", i), list(p), max_new_tokens)
        step_no = 0
        while sched.busy():
            entries, sampled = sched.schedule()
            logits = self.step(entries)
            if sampled:
                if sc.top_k == 1:
                    ids = ops.argmax_rows(logits)
                else:
                    ids = ops.sample(logits, top_k=sc.top_k, top_p=sc.top_p if sc.top_p > 0 else 1.0,
                                     temperature=sc.temperature, seed=sc.random_seed, step=step_no)
                sched.accept(sampled, ids.cpu().tolist(), sc.end_id)
            step_no += 1
        return [sched.finished[("gen", i)] for i in range(len(prompts))]


@dataclass
class _Request:
    seq_id: object
    prompt: list
    max_new: int
    fed: int = 0                       # prompt tokens already run
    out: list = field(default_factory=list)
    blocks: int = 0                    # pages promised to it at admission


class InflightScheduler:
    """Continuous batching: every step takes one token of each running sequence that is generating and fills the rest of
    the step's token budget with portions of the prompts still being read (oldest first).  A waiting request is admitted
    when a state slot is free and the pool can hold its prompt and all its new tokens beside what was promised to the
    running ones, so no admitted sequence ever has to be evicted."""

    def __init__(self, session: InflightSession, max_step_tokens: int = 512):
        self.s, self.budget = session, max(1, int(max_step_tokens))
        self.waiting, self.running, self.finished = deque(), [], {}
        self.promised = 0

    def add(self, seq_id, prompt, max_new):
        if not prompt:
            raise ValueError("empty prompt")
        self.waiting.append(_Request(seq_id, prompt, max_new))

    def busy(self):
        return bool(self.waiting or self.running)

    def _admit(self):
        m = self.s.kv_cache_manager
        while self.waiting and len(self.running) < self.s.slot_manager.slots:
            r = self.waiting[0]
            need = -(-(len(r.prompt) + r.max_new) // m.tokens_per_block)
            if need > m.blocks:
                raise RuntimeError(f"request {r.seq_id!r} needs {need} pages; the pool has {m.blocks}")
            if self.promised + need > m.blocks:
                break
            r.blocks, self.promised = need, self.promised + need
            self.running.append(self.waiting.popleft())

    def schedule(self):
        """-> (entries for InflightSession.step, [requests whose next token is sampled from this step's logits])."""
        self._admit()
        entries, sampled, left = [], [], self.budget
        for r in self.running:                                  # running decodes first: one token each
            if r.fed == len(r.prompt):
                entries.append((r.seq_id, [r.out[-1]], [0]))
                sampled.append(r)
                left -= 1
        for r in self.running:
            if r.fed < len(r.prompt) and left > 0:
                n = min(left, len(r.prompt) - r.fed)
                last = r.fed + n == len(r.prompt)
                entries.append((r.seq_id, r.prompt[r.fed:r.fed + n], [n - 1] if last else []))
                r.fed += n
                left -= n
                if last:
                    sampled.append(r)
        # rows of the logits follow the order of the entries
        order = {e[0]: k for k, e in enumerate(entries)}
        sampled.sort(key=lambda r: order[r.seq_id])
        return entries, sampled

    def accept(self, sampled, ids, end_id=None):
        for r, tok in zip(sampled, ids):
            r.out.append(int(tok))
            if len(r.out) >= r.max_new or (end_id is not None and tok == end_id):
                self.finished[r.seq_id] = r.out
                self.running.remove(r)
                self.promised -= r.blocks
                self.s.end(r.seq_id)
