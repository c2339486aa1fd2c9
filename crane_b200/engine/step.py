"""The step function: one batch of (request, its next tokens) through the model.

A batch may hold portions of prompts beside single decoded tokens, cut
anywhere.  Only the tokens given are run; everything earlier comes from the
cache.  The reference has two separate calls instead, one whole prompt of one
sequence (``forward``, crane-core/src/models/hunyuan_dense/modeling.rs:990-1066)
or one token of each of N sequences (``step_batch_decode``, :1225-1259), and
copies caches together and apart around the latter (:1150-1210, 1270-1311).

Per step the host builds one block of int32 metadata (token ids, positions,
the entry of each token, wanted rows, per entry the block-table row of every
layer group and the state slot), copies it to the device in one transfer and
runs the model's schedule.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheError, OutOfPages
from ..cache.pools import CachePools, bytes_per_page, group_layers
from ..config import EngineConfig, read_config_json, resolve
from ..config.engine_config import parse_memory_limit
from ..parts import DecoderModel, Runtime
from ..weights.loader import open_folder
from ..weights.safetensors_io import DictSource


# A decode step whose longest context is at most this many keys takes at most 8 key slices per
# (request, kv head), which merge in their cluster without a second kernel (see
# ``Kernels.decode_splits``).
SHORT_CONTEXT = 2048
SHORT_GRAPH_KEY = 1 << 20
# A step whose every entry has at most this many keys in all (whole short prompts).
SHORT_PROMPT = 64


@dataclass
class StepEntry:
    """A request's next tokens in this step and the places among them whose
    logits are wanted."""
    request_id: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepContext:
    """What the parts see of a step.  Device tensors are views into buffers
    whose addresses do not change from step to step."""
    n_tokens: int
    n_entries: int
    n_want: int
    max_q_len: int
    max_kv_len: int
    max_positions: int
    tokens: torch.Tensor        # int32 [n_tokens]
    positions: torch.Tensor     # int32 [n_tokens]
    tok_entry: torch.Tensor     # int32 [n_tokens]  index of the token's entry
    want_rows: torch.Tensor     # int32 [n_want]    rows whose logits are wanted
    cu_q: torch.Tensor          # int32 [n_entries + 1]  first row of each entry
    kv_len: torch.Tensor        # int32 [n_entries]  cached length after this step
    slots: torch.Tensor         # int32 [n_entries]  state slot of each entry
    block_tables: List[torch.Tensor]   # per layer group int32 [n_entries, max_blocks]
    # host copies for parts that plan on the host
    h_cu_q: np.ndarray
    h_kv_len: np.ndarray
    h_slots: np.ndarray
    deferred_tokens: torch.Tensor      # int32 [max entries]: what the last step sampled, row by row;
                                       # a token id <= -2 in ``tokens`` is read from row -id - 2
    graph_bucket: int = 0       # > 0: a decode step padded to this many entries
    real_entries: int = 0
    graph_key: Optional[tuple] = None   # a step with prompt portions whose rows are padded to a
                                        # multiple of 64 so that a captured graph fits it; the
                                        # padding rows have tok_entry -1 and belong to no entry,
                                        # padding entries have no rows and no cached length, and
                                        # the wanted rows beyond ``real_want`` repeat row 0
    real_want: int = 0
    replay: bool = False        # a step with a graph_key: replay its graph (else launch its kernels)
    single_entries: int = 0     # > 0: a step with prompt portions whose entries of exactly one token
                                # (decoded tokens, about this many) are worth a kernel of their own:
                                # an attention mixer may give them to its split-KV decode kernel and
                                # the rest to its prefill kernel
    short_prompts: bool = False     # no entry has more than 64 keys in all (whole short prompts)


class _MetaBuffers:
    """One pinned host block and one device block with the same fixed layout."""

    def __init__(self, cap_tokens: int, cap_entries: int, max_blocks: List[int], device):
        self.cap_tokens, self.cap_entries, self.max_blocks = cap_tokens, cap_entries, max_blocks
        off = 0
        self.off: Dict[str, int] = {}
        for name, size in (("tokens", cap_tokens), ("positions", cap_tokens),
                           ("tok_entry", cap_tokens), ("want_rows", cap_tokens),
                           ("cu_q", cap_entries + 1), ("kv_len", cap_entries),
                           ("slots", cap_entries)):
            self.off[name] = off
            off += (size + 3) // 4 * 4              # keep every array 16-byte aligned
        self.bt_off = []
        for mb in max_blocks:
            self.bt_off.append(off)
            off += (cap_entries * mb + 3) // 4 * 4
        self.total = off
        self.bt_off_arr = np.asarray(self.bt_off or [0], dtype=np.int32)
        self.max_blocks_arr = np.asarray(max_blocks or [0], dtype=np.int32)
        self.host = torch.empty(off, dtype=torch.int32).pin_memory()
        self.np = self.host.numpy()
        self.dev = torch.zeros(off, dtype=torch.int32, device=device)
        self.copied = torch.cuda.Event()
        self.copied.record()

    def view(self, name: str, n: int, device: bool):
        o = self.off[name]
        return (self.dev if device else self.np)[o:o + n]

    def table(self, g: int, n: int, device: bool):
        o, mb = self.bt_off[g], self.max_blocks[g]
        flat = (self.dev if device else self.np)[o:o + n * mb]
        return flat.view(n, mb) if device else flat.reshape(n, mb)


class ModelRunner:
    """Owns model, cache and buffers; ``step`` is the one way tokens get through."""

    def __init__(self, model_dir: Optional[str] = None, engine_config: Optional[EngineConfig] = None,
                 *, config: Optional[dict] = None, tensors=None, model_type: Optional[str] = None):
        self.cfg = engine_config or EngineConfig()
        if model_dir is not None:
            cfg_dict = read_config_json(model_dir)
            source, where = open_folder(model_dir), model_dir
        elif config is not None and tensors is not None:
            cfg_dict, source, where = config, DictSource(tensors), "the given tensors"
        else:
            raise ValueError("give a model folder, or a config dict with its tensors")
        arch = resolve(cfg_dict, model_type)
        self.model_config = arch.config_from_dict(cfg_dict)
        self.spec = arch.build_spec(self.model_config)
        dtype = torch.float32 if self.cfg.dtype == "float32" else torch.bfloat16
        self.max_seq_len = min(self.cfg.max_seq_len or self.spec.max_positions, self.spec.max_positions)
        self.cap_tokens = self.cfg.max_batched_tokens
        self.cap_entries = max(self.cfg.max_concurrent, 1)
        head_sizes = sorted({int(ps.params["head_dim"]) for layer in self.spec.layers
                             for ps in layer.parts.values() if "head_dim" in ps.params})
        self.rt = Runtime(self.cfg.device, dtype, self.cfg.workspace_rows or self.cap_tokens,
                          self.cap_entries, head_sizes)
        torch.cuda.set_device(self.rt.device)
        self.model = DecoderModel(self.spec, source, self.rt, where)
        self._build_cache()
        # the sampler writes here; the next step's embedding may read from it
        self.deferred_tokens = torch.zeros(self.cap_entries, dtype=torch.int32, device=self.rt.device)
        self.steps = 0
        # decode steps (one token per entry) of the bfloat16 path replay a captured graph
        self._graphs: Dict[object, tuple] = {}
        self._shape_seen: Dict[tuple, int] = {}      # how often a shape of small step has come
        self._graph_generation = -1
        has_state = any(n.kind == "state" for n in self.model.cache_needs())
        self._graphs_ok = (self.cfg.use_cuda_graphs and not self.rt.exact and self.model.capturable()
                           and (not has_state or self.model.state_graph_safe()))
        # Steps of single tokens are padded to a batch-size bucket (rows of no entry, entries without
        # rows) and replay that bucket's graph; with a mixer that keeps state they are padded as
        # steps with prompt portions are, to a shape of their own.
        self._pad_with_copies = not has_state
        self.graph_replays = 0
        self.graph_captures = 0                    # steps that ran kernel by kernel and were recorded for their shape
        self._step_done = torch.cuda.Event()       # recorded behind every step's kernels
        self._step_done.record()

    # ---- cache geometry -------------------------------------------------
    def _build_cache(self) -> None:
        needs = self.model.cache_needs()
        ps = self.cfg.page_size
        keys, _ = group_layers(needs)
        elem = 4 if self.rt.exact else 2
        per_page = bytes_per_page(needs, ps, elem)
        full = self.cap_entries * ((self.max_seq_len + ps - 1) // ps)    # every request at the limit
        if self.cfg.num_pages > 0:
            pages = self.cfg.num_pages
        elif self.cfg.max_cache_tokens > 0:
            pages = (self.cfg.max_cache_tokens + ps - 1) // ps
        else:
            free, total = torch.cuda.mem_get_info(self.rt.device)
            limit = parse_memory_limit(self.cfg.gpu_memory_limit, total)
            budget = int(free * 0.85)
            if limit > 0:
                budget = min(budget, max(0, limit - (total - free)))
            cost = max(1, sum(per_page))
            pages = max(1, min(full, budget // cost))
        self.pools = CachePools(needs, [pages] * len(keys), ps, self.cap_entries, self.rt.dtype,
                                self.rt.device)
        self.table = self.pools.table
        self.max_blocks = [(self.max_seq_len + ps - 1) // ps for _ in keys] or [1]
        self.meta = _MetaBuffers(self.cap_tokens, self.cap_entries, self.max_blocks if keys else [],
                                 self.rt.device)
        self.num_groups = len(keys)

    # ---- requests -------------------------------------------------------
    def is_live(self, rid: int) -> bool:
        return self.table.is_live(rid)

    def end(self, rid: int) -> None:
        """The request is finished: its pages and slot are given back."""
        self.table.release(rid)

    def length(self, rid: int) -> int:
        return self.table.length(rid)

    # ---- the step -------------------------------------------------------
    def prepare(self, entries: Sequence[StepEntry], reserved: bool = False) -> StepContext:
        """Takes pages for the step's tokens (unless the caller has: ``reserved``)
        and lays the metadata out on host and device.  A reserved step's tokens
        were checked on admission; it may name a token that the last step
        sampled and the host has not read yet as ``-(row + 2)``, ``row`` being
        the token's place in ``deferred_tokens``."""
        n_entries = len(entries)
        if n_entries == 0:
            raise ValueError("a step needs at least one entry")
        if n_entries > self.cap_entries:
            raise ValueError(f"{n_entries} entries in one step, the engine holds {self.cap_entries}")
        counts = [len(e.tokens) for e in entries]
        n_tokens = sum(counts)
        if min(counts) <= 0:
            raise ValueError("an entry without tokens")
        if n_tokens > self.cap_tokens:
            raise ValueError(f"{n_tokens} tokens in one step exceed max_batched_tokens={self.cap_tokens}")
        if len({e.request_id for e in entries}) != n_entries:
            raise ValueError("a request appears twice in one step")
        vocab = self.spec.vocab_size
        arrays = [np.asarray(e.tokens) for e in entries]
        if not reserved:
            # a caller that went through the scheduler has had its tokens checked on admission
            for e, c, t in zip(entries, counts, arrays):
                if t.min() < 0 or t.max() >= vocab:
                    raise ValueError(f"request {e.request_id}: token id outside [0, {vocab})")
        for e, c in zip(entries, counts):
            for w in e.want:
                if not 0 <= w < c:
                    raise ValueError(f"request {e.request_id}: wanted place {w} outside its {c} tokens")
        if not reserved:
            # check everything first, so that a refused step changes nothing
            ps = self.cfg.page_size
            need = [0] * self.num_groups
            new_requests = 0
            for e, c in zip(entries, counts):
                live = self.table.is_live(e.request_id)
                before = self.table.length(e.request_id) if live else 0
                if before + c > self.max_seq_len:
                    raise CacheError(f"request {e.request_id} would pass the sequence limit "
                                     f"{self.max_seq_len}")
                new_requests += 0 if live else 1
                for g in range(self.num_groups):
                    need[g] += (self.table.pages_needed(e.request_id, c, g) if live
                                else (c + ps - 1) // ps)
            if new_requests > self.table.free_slots():
                raise CacheError(f"{new_requests} new requests, {self.table.free_slots()} free slots")
            for g in range(self.num_groups):
                if need[g] > self.table.free_pages(g):
                    raise OutOfPages(f"the step needs {need[g]} pages of group {g}, "
                                     f"{self.table.free_pages(g)} are free")
            for e, c in zip(entries, counts):
                if not self.table.is_live(e.request_id):
                    self.table.admit(e.request_id)
                self.table.extend(e.request_id, c)
        # a pure decode step is padded to a fixed batch size so that a captured graph fits it
        pad_to = 0
        if (self._graphs_ok and self._pad_with_copies and max(counts) == 1
                and all(len(e.want) == 1 for e in entries)):
            pad_to = self._bucket(n_entries)
        # The entries run in the order of their cached lengths, longest first: the attention kernels'
        # CTAs go to the SMs in the order of the entries, and what is left for the end should be short.
        # Wanted rows are looked up through the order, so the logits come back in the caller's order.
        place = list(range(n_entries))              # place[i]: where the caller's entry i runs
        if n_entries >= 4:
            lengths = [self.table.length(e.request_id) for e in entries]
            order = sorted(range(n_entries), key=lambda i: -lengths[i])
            if order != place:
                for p, i in enumerate(order):
                    place[i] = p
                arrays = [arrays[i] for i in order]
                counts = [counts[i] for i in order]
        else:
            order = place
        m = self.meta
        m.copied.synchronize()                      # the last step's copy has left the host block
        real_entries = n_entries
        ids = np.fromiter((entries[i].request_id for i in order), dtype=np.int64, count=n_entries)
        cnt = np.asarray(counts, dtype=np.int32)
        # one native call lays out positions, entry of each token, cu_q, kv_len, slots, block tables
        n_tokens = self.table.fill_step(ids, cnt, m.np, m.off["positions"], m.off["tok_entry"],
                                        m.off["cu_q"], m.off["kv_len"], m.off["slots"], m.bt_off_arr,
                                        m.max_blocks_arr)
        # Decoded tokens beside prompt portions: when together they read enough cached keys, they are
        # worth the split-KV decode kernel (the prefill kernel would give each a whole query tile with
        # one live row and walk its context unsliced).
        # Whole prompts of at most 64 tokens each (nothing cached before them): the warp-level flash
        # attention, in tiles of 64 rows and several CTAs per SM, beats the tcgen05 kernel's 128-row
        # tiles there (see the attention part); it is part of a small step's shape, since a graph holds
        # the kernel it was recorded with.
        short_prompts = int(m.view("kv_len", n_entries, False).max()) <= SHORT_PROMPT
        singles = 0
        if not pad_to and not self.rt.exact:
            one = cnt == 1
            if one.any() and int(m.view("kv_len", n_entries, False)[one].sum()) >= self.cfg.mixed_decode_min_keys:
                singles = int(one.sum())
        # a small step with prompt portions: its rows are padded to a multiple of 64, its entries
        # and wanted places to a power of two, and from the second step of the same (rows,
        # entries, wanted, single-token entries) on a captured graph is replayed
        key = None
        # (a prompt portion alone or beside one other entry has few shapes, so all of them up to
        # graph_max_tokens are worth a graph; mixes of many entries come in many shapes, and only the
        # small ones, which the host could not launch as fast as the device runs them, get one)
        limit = self.cfg.graph_max_tokens if n_entries <= 2 else self.cfg.graph_max_tokens // 4
        if (not pad_to and self._graphs_ok and 0 < n_tokens <= limit):
            rows = min(-(-n_tokens // 64) * 64, self.cap_tokens)
            wanted = sum(len(e.want) for e in entries)
            shape = ("rows", rows, self._power_of_two(n_entries, self.cap_entries),
                     self._power_of_two(wanted, rows) if wanted else 0,
                     self._power_of_two(singles, self.cap_entries) if singles else 0,
                     1 if short_prompts else 0)
            seen = self._shape_seen.get(shape, 0) + 1
            self._shape_seen[shape] = seen
            if seen >= 2:
                key = shape
                singles = shape[4]
        m.view("tokens", n_tokens, False)[:] = arrays[0] if len(arrays) == 1 else np.concatenate(arrays)
        # A decode step is filled up to its bucket, a small step with prompt portions to its shape, with
        # rows that belong to no entry (they write nothing into a cache) and entries without rows (no
        # attention kernel has work for them): the padding costs the products' rows and nothing else.
        # (Copies of a real entry, as decode steps were once padded with, read that entry's keys again:
        # 40 requests in a bucket of 64 took the time of 64.)
        pad_rows = pad_to if pad_to else (key[1] if key is not None else 0)
        pad_entries = pad_to if pad_to else (key[2] if key is not None else 0)
        if pad_rows > n_tokens:
            m.view("tokens", pad_rows, False)[n_tokens:] = 0
            m.view("positions", pad_rows, False)[n_tokens:] = 0
            m.view("tok_entry", pad_rows, False)[n_tokens:] = -1
            n_tokens = pad_rows
        cu = m.view("cu_q", n_entries + 1, False)
        kvl = m.view("kv_len", n_entries, False)
        slots = m.view("slots", n_entries, False)
        if pad_entries > n_entries:
            last = int(cu[n_entries])
            cu = m.view("cu_q", pad_entries + 1, False)
            kvl = m.view("kv_len", pad_entries, False)
            slots = m.view("slots", pad_entries, False)
            cu[n_entries + 1:] = last
            kvl[n_entries:] = 0
            slots[n_entries:] = 0
            n_entries = pad_entries
        if pad_to:
            n_want = pad_to
            rows_of = m.view("want_rows", n_want, False)
            rows_of[:real_entries] = np.asarray(place, dtype=np.int32)    # one row per entry
            rows_of[real_entries:] = np.arange(real_entries, n_want, dtype=np.int32)
        else:
            want_rows = [int(cu[place[i]]) + w for i, e in enumerate(entries) for w in e.want]
            n_want = real_want = len(want_rows)
            if key is not None and key[3] > n_want:
                want_rows += [0] * (key[3] - n_want)        # more rows of logits than are wanted
                n_want = key[3]
            if n_want:
                m.view("want_rows", n_want, False)[:] = np.asarray(want_rows, dtype=np.int32)
        m.dev.copy_(m.host, non_blocking=True)
        m.copied.record()

        ctx = StepContext()
        ctx.graph_bucket, ctx.real_entries = pad_to, real_entries
        ctx.graph_key = key
        ctx.single_entries = singles
        ctx.short_prompts = short_prompts
        # While the device still runs the step before, the host launches this step's kernels
        # behind it at no cost, and launched one by one they ran a little faster than replayed
        # (a serving mix: 5 % per step): a graph pays when the device waits for the host.  The
        # step is padded to its shape either way, so that both ways run the same kernels on the
        # same rows and give the same bits.
        ctx.replay = key is not None and self._step_done.query()
        ctx.real_want = n_want if key is None else real_want
        ctx.n_tokens, ctx.n_entries, ctx.n_want = n_tokens, n_entries, n_want
        # a padded step never counts as one of single tokens only: its filling entries have none
        ctx.max_q_len = int(cnt.max()) if key is None else max(2, int(cnt.max()))
        ctx.max_kv_len = int(kvl.max())
        ctx.max_positions = self.max_seq_len
        ctx.deferred_tokens = self.deferred_tokens
        ctx.tokens = m.view("tokens", n_tokens, True)
        ctx.positions = m.view("positions", n_tokens, True)
        ctx.tok_entry = m.view("tok_entry", n_tokens, True)
        ctx.want_rows = m.view("want_rows", n_want, True)
        ctx.cu_q = m.view("cu_q", n_entries + 1, True)
        ctx.kv_len = m.view("kv_len", n_entries, True)
        ctx.slots = m.view("slots", n_entries, True)
        ctx.block_tables = [m.table(g, n_entries, True) for g in range(self.num_groups)]
        ctx.h_cu_q = cu.copy()
        ctx.h_kv_len = kvl.copy()
        ctx.h_slots = slots.copy()
        return ctx

    def step(self, entries: Sequence[StepEntry], reserved: bool = False) -> torch.Tensor:
        """Runs the entries as one batch and returns float logits
        [number of wanted places, vocab] on the device, in the order of the
        entries and of their ``want``."""
        ctx = self.prepare(entries, reserved)
        self.steps += 1
        try:
            if ctx.graph_bucket:
                # (a graph holds the number of key slices its attention was recorded with: short
                # contexts, which take fewer, have graphs of their own)
                short = ctx.max_kv_len <= SHORT_CONTEXT
                return self._replay(ctx, ctx.graph_bucket + (SHORT_GRAPH_KEY if short else 0))[:ctx.real_entries]
            if ctx.graph_key is not None and ctx.replay:
                return self._replay(ctx, ctx.graph_key)[:ctx.real_want]
            return self.model.forward(ctx, self.pools.layers)[:ctx.real_want]
        finally:
            self._step_done.record()

    # ---- captured decode steps -----------------------------------------
    def _bucket(self, n: int) -> int:
        """The batch size a decode step of ``n`` entries is padded to: the next power
        of two up to 16, finer steps above, or the most entries a step can have
        where that is less."""
        b = 1
        while b < n:
            b *= 2
        if b > 16:
            # above 16 in steps of a sixteenth of the power of two (20, 24, 28, 32, 36, 40, ..., 64, 72, 80,
            # ...): the attention's number of key slices is chosen for the bucket, and what suits 64
            # requests suits neither 36 nor 40 (measured at 4 kv heads and a context of 8,192: 36
            # requests 5.94 ms per step with one slice, 4.76 ms with two; 40 requests 5.90 and 6.55 ms)
            step = max(4, b // 16)
            b = -(-n // step) * step
        return min(b, self.cap_entries)

    MAX_SHAPE_GRAPHS = 256      # graphs of small steps kept; the least recently used one goes first

    @staticmethod
    def _power_of_two(n: int, cap: int) -> int:
        b = 1
        while b < n:
            b *= 2
        return min(b, cap)

    def _replay(self, ctx: StepContext, key) -> torch.Tensor:
        if self._graph_generation != self.rt.ws.generation:
            self._graphs.clear()                    # a buffer moved: captured addresses are stale
            self._graph_generation = self.rt.ws.generation
        entry = self._graphs.pop(key, None)
        if entry is None and isinstance(key, tuple):
            shapes = [k for k in self._graphs if isinstance(k, tuple)]
            if len(shapes) >= self.MAX_SHAPE_GRAPHS:
                del self._graphs[shapes[0]]
                # a capture costs more than two steps launched kernel by kernel: a shape that was
                # dropped has to come ten times more before it is captured again
                self._shape_seen[shapes[0]] = -8
        if entry is None:
            # once eagerly, so that every buffer exists; then the same step again under capture
            # (nothing runs while it is recorded)
            eager = self.model.forward(ctx, self.pools.layers)
            if self._graph_generation != self.rt.ws.generation:
                self._graphs.clear()
                self._graph_generation = self.rt.ws.generation
            before = self.rt.launches
            torch.cuda.synchronize(self.rt.device)
            graph = torch.cuda.CUDAGraph()
            try:
                with torch.cuda.graph(graph):
                    logits = self.model.forward(ctx, self.pools.layers)
            except Exception as exc:
                # the step itself has run (kernel by kernel, above); what is lost is the process's
                # further use of captures, which an aborted one leaves in an undefined state
                raise RuntimeError(
                    "a step could not be recorded as a CUDA graph; a part that reads results on the "
                    "host in its forward must set `capturable = False` (or run the engine with "
                    "use_cuda_graphs=False)") from exc
            # The step itself has just run, kernel by kernel; the graph serves the later steps of its
            # shape.  (Replaying it now as well would run the step twice, which pages bear, since the
            # same rows get the same values, but a mixer's per-request state does not.)
            self._graphs[key] = (graph, logits, self.rt.launches - before)
            self.rt.launches = before
            self.graph_captures += 1
            return eager
        self._graphs[key] = entry                   # (back) at the end: the most recently used
        graph, logits, launches = entry
        graph.replay()
        self.rt.launches += launches
        self.graph_replays += 1
        return logits
