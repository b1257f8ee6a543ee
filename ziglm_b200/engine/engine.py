"""The engine: a model on one GPU, its cache, and the one step function everything goes through.

Names follow the reference's library surface (src/root.zig:22-35): ``Engine``
with ``load`` (src/engine.zig:64), ``prefill`` (321), ``decode`` (345),
``generate`` (382) and ``reset`` (287); ``EngineOptions`` (src/engine.zig:32-37).
The reference serves one sequence; here ``step`` takes a batch of sequences that
either all start at their first token or all go on, each with its own length,
runs exactly the tokens it is given from the cache earlier steps left, and
returns the logits at the wanted places.  ``prefill``/``decode``/``reset`` are the
reference's single-sequence calls expressed through ``step``.
"""
from __future__ import annotations

import gc
import weakref
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels
from ..cache import CacheStorage, PAGE_SIZE
from ..config import config_from_dict, config_from_folder
from ..weights import load_tensors, random_tensors
from .batch import BatchLayout, StepContext, pack_batch, views
from .model import Model, declare_parameters
from .workspace import Workspace


class StepError(ValueError):
    """The step was asked for something it cannot run (empty sequence, unknown token, ...)."""


@dataclass
class EngineOptions:
    """Options of ``Engine.load``; the first four are the reference's (src/engine.zig:32-37).

    num_threads  accepted and ignored (the reference's CPU worker count).
    max_seq_len  positions one sequence may hold; default min(max_position_embeddings, 4096),
                 the reference's choice (src/engine.zig:207).
    seed         seed of sampling (and of random weights when there is no folder).
    use_gpu      must stay true: there is no CPU path.
    dtype        "bfloat16" (the kernels and precisions of serving) or "float32" (everything in true 32-bit).
    max_tokens   positions the cache holds for all live sequences together, each sequence rounded up to
                 whole pages of 64; default max_batch * max_seq_len.
    max_batch    most sequences alive at once (slots).
    device       CUDA device.
    beyond_max_positions  let ``max_seq_len`` pass the model's max_position_embeddings: the rotation is a function
                 of the position alone, so the arithmetic is defined there; what a model makes of positions it was
                 not trained on is its user's concern (replay, which checks arithmetic, sets it).
    """
    num_threads: Optional[int] = None
    max_seq_len: Optional[int] = None
    seed: int = 42
    use_gpu: bool = True
    dtype: str = "bfloat16"
    max_tokens: Optional[int] = None
    max_batch: int = 8
    device: str = "cuda:0"
    use_graphs: bool = True
    beyond_max_positions: bool = False


_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "f32": torch.float32,
           "fp32": torch.float32}


def _require_cuda(device: str) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("ziglm_b200 needs a CUDA device (sm_100a); there is no CPU path")
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError(f"ziglm_b200 runs on CUDA devices only, not on {device!r}")
    return dev


class Engine:
    def __init__(self, config, model: Model, options: EngineOptions):
        self.config = config
        self.model = model
        self.options = options
        self.spec = model.spec
        self.device = model.device
        self.dtype = model.dtype
        limit = self.spec.max_positions or 4096
        self.max_seq_len = int(options.max_seq_len) if options.max_seq_len else min(limit, 4096)
        if self.spec.max_positions and self.max_seq_len > self.spec.max_positions and not options.beyond_max_positions:
            raise ValueError(f"max_seq_len {self.max_seq_len} exceeds the model's max_position_embeddings "
                             f"{self.spec.max_positions}")
        max_tokens = options.max_tokens or options.max_batch * (-(-self.max_seq_len // PAGE_SIZE) * PAGE_SIZE)
        n_slots = max(1, min(options.max_batch, -(-max_tokens // PAGE_SIZE)))
        kv, reads, state = model.cache_plan()
        self.cache = CacheStorage(kv, reads, state, max_tokens, n_slots, self.max_seq_len, self.dtype, self.device)
        self.ws = Workspace(self.device)
        self.graph_ws = Workspace(self.device)     # scratch of the captured decode steps, shared by all batch sizes
        self._host = [None, None]
        self._host_events = [None, None]
        self._dev: Optional[torch.Tensor] = None
        self._flip = 0
        self._graphs: Dict[int, "_DecodeGraph"] = {}
        self._repeat: Optional["_RepeatedDecode"] = None      # the last decode step, ready to be taken once more
        self._graph_kernels = 0
        self.last_step_h2d_bytes = 0
        self._default_slot: Optional[int] = None
        kernels.require(model.kernel_libraries())

    # ---------------------------------------------------------------- creation
    @classmethod
    def load(cls, model_path: str, options: Optional[EngineOptions] = None) -> "Engine":
        """Load a model folder (config.json + model.safetensors); the class of model is chosen by config.json."""
        options = options or EngineOptions()
        if not options.use_gpu:
            raise RuntimeError("use_gpu=False: there is no CPU path in this library")
        device = _require_cuda(options.device)
        dtype = _DTYPES[options.dtype]
        if os.path.isfile(model_path):
            model_path = os.path.dirname(os.path.abspath(model_path))
        config = config_from_folder(model_path)
        spec = config.model_spec()
        declared = declare_parameters(spec)
        torch.cuda.set_device(device)
        tensors = load_tensors(model_path, declared, dtype, device)
        model = Model(spec, dtype, device)
        model.bind(tensors)
        return cls(config, model, options)

    @classmethod
    def from_config(cls, config, options: Optional[EngineOptions] = None, std: float = 0.02,
                    norm_jitter: float = 0.0) -> "Engine":
        """A model with random weights made on the device from ``options.seed`` (no files)."""
        options = options or EngineOptions()
        device = _require_cuda(options.device)
        dtype = _DTYPES[options.dtype]
        if isinstance(config, dict):
            config = config_from_dict(config)
        spec = config.model_spec()
        declared = declare_parameters(spec)
        torch.cuda.set_device(device)
        tensors = dict(random_tensors(declared, options.seed, dtype, device, std, norm_jitter))
        model = Model(spec, dtype, device)
        model.bind(tensors)
        return cls(config, model, options)

    # ------------------------------------------------------------------- slots
    def alloc_slot(self) -> int:
        self._repeat = None
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self._repeat = None
        self.cache.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.slots.length_of(slot)

    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    # -------------------------------------------------------------------- step
    def step(self, entries: Sequence[Tuple[int, Sequence[int]]],
             want: Optional[Sequence[Sequence[int]]] = None,
             device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run one step.

        entries  (slot, tokens) per sequence: the next tokens of that sequence, at least one.
        want     per sequence, the places among its tokens whose logits are wanted
                 (default: the last token of each).
        device_tokens  int32 on the device, one id per sequence in the order of the entries: the tokens of a
                 step of one token each, when the host does not know them yet (ids that a sampling kernel
                 earlier in the stream has written, or will have by the time this step's kernels run).  The ids in
                 ``entries`` are then place holders (give 0).  The generation loop uses this to launch a step
                 before it has read the ids of the step before.
        Returns float32 logits [n_wanted, vocab] on the device, in the order of the entries
        and of ``want``, or None if nothing is wanted.  The tensor is scratch of the engine:
        it is overwritten by the next step.
        """
        if not entries:
            raise StepError("a step needs at least one sequence")
        if device_tokens is not None:
            if any(len(t) != 1 for _, t in entries):
                raise StepError("tokens from the device are for steps of one token per sequence")
            if (not device_tokens.is_cuda or device_tokens.dtype != torch.int32 or device_tokens.dim() != 1
                    or device_tokens.numel() < len(entries)):
                raise StepError("device_tokens must be int32 on the device, one id per sequence")
        if want is None and self._repeat is not None:
            logits = self._repeat_decode(entries, device_tokens)
            if logits is not None:
                return logits
        self._repeat = None
        slots = [int(s) for s, _ in entries]
        new_tokens = [list(t) for _, t in entries]
        if len(set(slots)) != len(slots):
            raise StepError("a slot appears twice in one step")
        V = self.spec.vocab_size
        for s, toks in zip(slots, new_tokens):
            if not toks:
                raise StepError(f"slot {s}: a sequence must bring at least one token")
            for t in toks:
                if not (0 <= int(t) < V):
                    raise StepError(f"slot {s}: token {t} is outside the vocabulary of {V}")
        past = [self.cache.slots.length_of(s) for s in slots]
        if want is None:
            want = [[len(t) - 1] for t in new_tokens]
        if len(want) != len(entries):
            raise StepError("`want` needs one list per sequence")
        want_rows: List[int] = []
        start = 0
        for toks, w in zip(new_tokens, want):
            for i in w:
                if not (0 <= int(i) < len(toks)):
                    raise StepError(f"wanted place {i} is outside the {len(toks)} tokens of its sequence")
                want_rows.append(start + int(i))
            start += len(toks)

        growth = {s: len(t) for s, t in zip(slots, new_tokens)}
        self.cache.slots.reserve(growth)

        T = start
        B = len(slots)
        single = all(len(t) == 1 for t in new_tokens)
        max_total = max(p + len(t) for p, t in zip(past, new_tokens))
        if single and want_rows == list(range(B)) and self.options.use_graphs:
            logits = self._graph_step(slots, past, new_tokens, want_rows, device_tokens)
            self.cache.slots.advance(growth)
            self._arm_repeat(slots, want is None or all(list(w) == [0] for w in want))
            return logits
        width = -(-max_total // self.cache.page_size)
        widths = tuple(width for _ in self.cache.groups)
        layout = BatchLayout(T, B, len(want_rows), widths)
        tables = [self.cache.block_table_rows(g, slots, width) for g in range(len(self.cache.groups))]

        host, dev = self._buffers(layout.total)
        pack_batch(layout, host, slots, past, new_tokens, want_rows, tables)
        dev[:layout.total].copy_(host[:layout.total], non_blocking=True)
        self._feed_tokens(dev, layout, device_tokens)
        self._host_events[self._flip].record()
        self.last_step_h2d_bytes = layout.total * 4
        step = self._context(layout, dev, single, max(len(t) for t in new_tokens), max_total, self.ws, past,
                             [len(t) for t in new_tokens], slots)
        logits = self.model.forward(step)
        self.cache.slots.advance(growth)
        return logits

    def _context(self, layout: BatchLayout, dev: torch.Tensor, single: bool, max_new: int, max_total: int,
                 ws: Workspace, past: List[int], new_lens: List[int], slots: List[int]) -> StepContext:
        v = views(layout, dev)
        step = StepContext(
            n_tokens=layout.n_tokens, n_seqs=layout.n_seqs, n_want=layout.n_want, tokens=v["tokens"],
            positions=v["positions"], seq_of_token=v["seq_of_token"], cu_seqlens=v["cu_seqlens"],
            past_lens=v["past_lens"], total_lens=v["total_lens"], slots=v["slots"], want_rows=v["want_rows"],
            block_tables=v["block_tables"], single_token=single, max_new=max_new, max_total=max_total,
            dtype=self.dtype, device=self.device, ws=ws, host_past_lens=past, host_new_lens=new_lens,
            host_slots=slots)
        step.io = [self.cache.io_for(place, step.block_tables) for place in range(len(self.spec.schedule))]
        return step

    # ------------------------------------------------------- decode steps as CUDA graphs
    @staticmethod
    def _feed_tokens(dev: torch.Tensor, layout: BatchLayout, device_tokens: Optional[torch.Tensor]) -> None:
        """Overwrite the token ids of a packed step on the device with ids that are already there."""
        if device_tokens is not None:
            at = layout.offsets["tokens"]
            dev[at:at + layout.n_tokens].copy_(device_tokens[:layout.n_tokens], non_blocking=True)

    def _graph_step(self, slots: List[int], past: List[int], new_tokens: List[List[int]],
                    want_rows: List[int], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """A step in which every sequence brings one token and every logit row is wanted: the launches of
        such a step depend on the batch size alone (everything else is read from device memory), so they are
        captured once per batch size and replayed (the reference does this for its one sequence,
        src/cuda_model.zig:1017-1069)."""
        B = len(slots)
        g = self._graphs.get(B)
        if g is None:
            g = _DecodeGraph(self, B)
            self._graphs[B] = g
        width = self.cache.max_pages_per_seq
        tables = [self.cache.block_table_rows(gi, slots, width) for gi in range(len(self.cache.groups))]
        host = g.staging()
        pack_batch(g.layout, host, slots, past, new_tokens, want_rows, tables)
        g.dev.copy_(host, non_blocking=True)
        self._feed_tokens(g.dev, g.layout, device_tokens)
        g.mark_copied()
        self.last_step_h2d_bytes = g.layout.total * 4
        return g.run(past, slots)

    # ---------------------------------------------- the same decode step once more
    def _arm_repeat(self, slots: List[int], plain_want: bool) -> None:
        """After a decode step of a batch: if the same sequences bring one token each again, nothing of the
        step's integers changes but the tokens, the lengths and, for a sequence that stands at a page boundary,
        one entry of its block table, as long as no group lets pages go behind a window and no sequence
        reaches its limit."""
        self._repeat = None
        if not plain_want or any(g.pages.window is not None for g in self.cache.groups):
            return
        lengths = np.array([self.cache.slots.length_of(s) for s in slots], dtype=np.int64)
        left = self.max_seq_len - int(lengths.max())
        if left <= 0:
            return
        g = self._graphs[len(slots)]
        self._repeat = _RepeatedDecode(list(slots), g, g.host[g.flip].numpy().copy(), left, lengths)

    def _repeat_decode(self, entries, device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        r = self._repeat
        if len(entries) != len(r.slots) or r.left <= 0:
            return None
        tokens = []
        for (slot, toks), known in zip(entries, r.slots):
            if slot != known or len(toks) != 1:
                return None
            tokens.append(toks[0])
        if min(tokens) < 0 or max(tokens) >= self.spec.vocab_size:
            return None                                   # the general path names the offender
        g, o, B = r.graph, r.graph.layout.offsets, len(tokens)
        image, page = r.image, self.cache.page_size
        at_boundary = np.nonzero(r.lengths % page == 0)[0]
        if at_boundary.size:
            # these sequences start a page with this token: take the pages (all or none) and enter them
            self.cache.slots.reserve({r.slots[b]: 1 for b in at_boundary})
            for gi, grp in enumerate(self.cache.groups):
                width = g.layout.table_widths[gi]
                for b in at_boundary:
                    idx = int(r.lengths[b]) // page
                    image[o[f"table{gi}"] + int(b) * width + idx] = grp.pages.pages_of[r.slots[b]][idx]
        image[o["tokens"]:o["tokens"] + B] = tokens
        for name in ("positions", "past_lens", "total_lens"):
            image[o[name]:o[name] + B] += 1
        host = g.staging()
        host.numpy()[:] = image
        g.dev.copy_(host, non_blocking=True)
        self._feed_tokens(g.dev, g.layout, device_tokens)
        g.mark_copied()
        self.last_step_h2d_bytes = g.layout.total * 4
        g.graph.replay()
        self._graph_kernels += g.kernels_per_replay
        length = self.cache.slots.length
        for slot in r.slots:
            length[slot] += 1
        r.lengths += 1
        r.left -= 1
        return g.logits

    # ------------------------------------------------------------- kernel health
    def check_kernels(self, read=None) -> None:
        """Raise :class:`~ziglm_b200.kernels.KernelError` if a bounded wait ran out inside a tensor-core kernel
        since the last check.  Such a kernel returned early: the rows of its step are not to be trusted, and the
        flat decode attention may have left its per-sequence counters non-zero.  Before raising, the counters of
        every workspace are zeroed and the decode step kept for repetition is dropped, so that the engine can be
        used again; the sequences that were live should be ended.  ``read``: a stand-in for
        ``kernels.wait_errors`` (tests).  Synchronises the device."""
        codes = (read or kernels.wait_errors)()
        if not any(codes.values()):
            return
        self._repeat = None
        for ws in (self.ws, self.graph_ws):
            ws.zero("attn_flat_counters")
        raise kernels.KernelError("a bounded wait ran out inside a kernel, the step's results are not valid: "
                                  + kernels.describe_wait_errors(codes))

    def graph_launched_kernels(self) -> int:
        """Kernels launched by graph replays since the counter was last read."""
        n, self._graph_kernels = self._graph_kernels, 0
        return n

    def _buffers(self, n: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """A pinned staging buffer that no copy in flight still reads, and the device buffer."""
        self._flip ^= 1
        i = self._flip
        if self._host[i] is None or self._host[i].numel() < n:
            cap = max(1024, 1 << (n - 1).bit_length())
            self._host[i] = torch.empty(cap, dtype=torch.int32).pin_memory()
            self._host_events[i] = torch.cuda.Event()
        else:
            self._host_events[i].synchronize()
        if self._dev is None or self._dev.numel() < n:
            cap = max(1024, 1 << (n - 1).bit_length())
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        return self._host[i], self._dev

    # ---------------------------------------- the reference's single-sequence calls
    def reset(self) -> None:
        """Forget the sequence of ``prefill``/``decode`` (the reference rewinds its one cache, src/engine.zig:287)."""
        if self._default_slot is not None:
            self.free_slot(self._default_slot)
            self._default_slot = None

    def prefill(self, tokens: Sequence[int]) -> torch.Tensor:
        """Run a whole prompt for the engine's own sequence; logits of its last token, float32 [vocab]."""
        if len(tokens) == 0:
            raise StepError("the prompt is empty")
        if self._default_slot is None:
            self._default_slot = self.alloc_slot()
        return self.step([(self._default_slot, tokens)])[0]

    def decode(self, token: int, pos: int) -> torch.Tensor:
        """Run one more token of the engine's own sequence at position ``pos``; its logits."""
        if self._default_slot is None:
            self._default_slot = self.alloc_slot()
        have = self.length(self._default_slot)
        if pos != have:
            raise StepError(f"decode at position {pos}, but the sequence holds {have} tokens")
        return self.step([(self._default_slot, [int(token)])])[0]

    def generate(self, prompts, options=None, callback=None):
        from .generate import generate
        return generate(self, prompts, options, callback)


@dataclass
class _RepeatedDecode:
    """A decode step that may be taken again as it is: its sequences, its graph, the packed integers of the
    step that was just run (as they lie in the staging buffer) and how many more steps keep them valid."""
    slots: List[int]
    graph: "_DecodeGraph"
    image: "object"
    left: int
    lengths: "object"        # int64 array: the sequences' lengths


class _DecodeGraph:
    """The captured launches of a decode step of one batch size, with the memory they point to."""

    def __init__(self, engine: Engine, batch: int):
        self._engine = weakref.ref(engine)      # the engine owns this object: no cycle, both go when it is dropped
        self.batch = batch
        width = engine.cache.max_pages_per_seq
        self.layout = BatchLayout(batch, batch, batch, tuple(width for _ in engine.cache.groups))
        self.dev = torch.empty(self.layout.total, dtype=torch.int32, device=engine.device)
        self.host = [torch.empty(self.layout.total, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.events = [torch.cuda.Event(), torch.cuda.Event()]
        self.used = [False, False]
        self.flip = 0
        self.ws = engine.graph_ws               # shared: steps run one after another, and so do replays
        self.ws_moves = -1                      # ``ws.moves`` when the launches were captured
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.kernels_per_replay = 0

    @property
    def engine(self) -> Engine:
        e = self._engine()
        if e is None:
            raise RuntimeError("the engine of this decode graph is gone")
        return e

    def staging(self) -> torch.Tensor:
        self.flip ^= 1
        if self.used[self.flip]:
            self.events[self.flip].synchronize()
        return self.host[self.flip]

    def mark_copied(self) -> None:
        self.events[self.flip].record()
        self.used[self.flip] = True

    def _context(self, past: List[int], slots: List[int]) -> StepContext:
        e = self.engine
        return e._context(self.layout, self.dev, True, 1, e.max_seq_len, self.ws, past, [1] * self.batch, slots)

    def run(self, past: List[int], slots: List[int]) -> torch.Tensor:
        e = self.engine
        if self.graph is not None and self.ws_moves == self.ws.moves:
            self.graph.replay()
            e._graph_kernels += self.kernels_per_replay
            return self.logits
        # First step of this batch size, or a larger batch has since made the shared scratch grow and move: run
        # the step as it is (this also sizes the scratch), then capture it.
        self.graph = None
        step = self._context(past, slots)
        before = kernels.launches()
        logits = e.model.forward(step)
        self.kernels_per_replay = kernels.launches() - before
        torch.cuda.current_stream().synchronize()
        graph = torch.cuda.CUDAGraph()
        # Nothing may destroy another graph while this one is being captured: an engine dropped earlier takes
        # its graphs with it only when the collector runs, and that must not be in the middle of the capture.
        gc.collect()
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph):
                captured = e.model.forward(self._context(past, slots))
        finally:
            if collecting:
                gc.enable()
        kernels.reset_launches_by(self.kernels_per_replay)
        assert captured.data_ptr() == logits.data_ptr()
        self.graph, self.logits, self.ws_moves = graph, logits, self.ws.moves
        return logits
