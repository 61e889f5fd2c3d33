"""ModelRunner: the model, its cache and the one step function.

``step(entries)`` takes a batch of (request, its next tokens, wanted places),
portions of prompts beside single decoded tokens, cut anywhere; it runs only the
tokens it is given, as one batch, against the cache earlier steps left, and
returns the logits at the wanted places as a device tensor ``[wanted, vocab]``
in the order of the entries and of their wanted places.  The scheduler, the
Python entry point and trace replay all drive this same function.

The reference's counterpart runs prompts and decode tokens as two forwards and
returns host vectors (models/llama/llama_model.cpp:298-726; app/main.cpp:295-337).
"""
from __future__ import annotations

import array
import gc
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..config.specs import ModelSpec
from ..models.decoder import DecoderModel
from ..parts.base import Runtime
from ..registry import architecture_of, read_config_json
from ..weights.loader import load_checkpoint
from .batch import ContextBuilder, StepContext, StepEntry


class OutOfPages(RuntimeError):
    """The cache pool cannot hold the tokens a step brings."""


_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        return dtype
    try:
        return _DTYPES[str(dtype)]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {dtype!r}") from None


def _build_model(spec: ModelSpec, rt: Runtime, arch=None):
    build = getattr(arch, "build", None) if arch is not None else None
    return build(spec, rt) if build else DecoderModel(spec, rt)


def _token_array(tokens) -> Optional[np.ndarray]:
    """The tokens as an int32 array; None if one does not fit 32 bits.  A list of thousands of
    Python ints goes through ``array``, which converts it several times faster than numpy does."""
    if isinstance(tokens, np.ndarray):
        if tokens.dtype == np.int32:
            return tokens
        if tokens.size and not (-2 ** 31 <= int(tokens.min()) and int(tokens.max()) < 2 ** 31):
            return None
        return tokens.astype(np.int32)
    try:
        return np.frombuffer(array.array("i", tokens), dtype=np.int32)
    except OverflowError:
        return None
    except TypeError:
        a = np.asarray(tokens)
        if a.dtype.kind not in "iu":
            raise
        return _token_array(a)


def expected_tensors_of(spec: ModelSpec) -> Dict[str, Tuple[Tuple[int, ...], str, str]]:
    """Checkpoint name -> (shape, role, init) of every tensor a model of ``spec`` needs."""
    shell = DecoderModel(spec, Runtime("cpu", torch.float32, ops=object()))
    return {n: (ps.shape, ps.role, ps.init) for n, (_, _, ps) in shell.expected_tensors().items()}


class _StepGraph:
    """What a captured step of one shape (the entries' token counts and wanted places) keeps: its
    metadata buffer at a fixed address, the captured graph and the logits tensor the graph writes."""

    def __init__(self, n_requests: int, n_tokens: int, n_wanted: int, n_groups: int, page_size: int, device):
        # block-table cells changed per step: new pages of the step's tokens, pages given back
        self.cap = 2 * n_requests + n_tokens // page_size + 8
        n = 3 * n_tokens + (n_requests + 1) + 2 * n_requests + n_wanted + n_groups * (1 + 2 * self.cap) \
            + 2 * n_requests                             # and which tokens come from the device
        self.meta = torch.zeros(n, dtype=torch.int32, device=device)
        self.graph = None
        self.logits: Optional[torch.Tensor] = None
        self.after_result = None                         # what the step's ``after`` returned at capture
        self.warm = 0


class ModelRunner:
    def __init__(self, model_dir: Optional[str] = None, *, config=None,
                 tensors: Optional[Dict[str, torch.Tensor]] = None,
                 dtype="bfloat16", device="cuda:0", page_size: int = 16,
                 num_pages: int = 1024, max_requests: int = 64,
                 max_tokens_per_step: int = 2048, max_model_len: Optional[int] = None,
                 ops=None, verbose: bool = False, cuda_graphs: bool = True):
        """Either ``model_dir`` (config.json + safetensors) or ``config`` + ``tensors``
        (checkpoint names -> tensors, e.g. from ``random_tensors``)."""
        self.dtype = parse_dtype(dtype)
        arch = None
        if config is None:
            cfg_dict = read_config_json(model_dir)
            arch = architecture_of(cfg_dict)
            config = arch.config_cls.from_dict(cfg_dict)
        self.config = config
        self.spec: ModelSpec = config.to_model_spec()
        self.rt = Runtime(device, self.dtype, ops=ops, page_size=page_size)
        self.model = _build_model(self.spec, self.rt, arch)
        if ops is None:
            # compile (first call) and load what this model needs; raises if it cannot
            self.rt.ops.prepare(self.model.required_kernels() + ["cache_table"],
                                verbose=verbose)

        expected = self.model.expected_tensors()
        if tensors is None:
            tensors = load_checkpoint(
                model_dir, {n: (ps.shape, ps.role) for n, (_, _, ps) in expected.items()},
                self.spec.ignorable)
        self.model.load_tensors(tensors)

        self.page_size = page_size
        if max_model_len is None:
            max_model_len = num_pages * page_size
        self.max_model_len = max_model_len
        self.max_requests = max_requests
        self.max_tokens_per_step = max_tokens_per_step
        self.cache = CacheManager(self.model.cache_specs(), page_size, num_pages, max_requests,
                                  -(-max_model_len // page_size), rt=self.rt)
        self._ctx = ContextBuilder(self.rt.device, max_tokens_per_step, max_requests)
        self.steps = 0
        self.tokens_run = 0
        # decode-only steps are captured once per batch size and replayed (no per-kernel launch
        # cost); only if every part launches the same kernels whatever the host-side values are
        # The same holds for a step with prompt portions whose shape (token count and wanted places
        # of every entry) comes again: whole prompts of one length, the full portions of a long
        # prompt.  Such a shape is captured when it is seen for the third time; the most recent
        # ``max_shape_graphs`` are kept (each holds the activations of its step).  Only steps of
        # at most ``shape_graph_entries`` entries are: a prompt or a portion alone in its step is
        # where the host's launches show (nothing is queued ahead of it), and where shapes come
        # again; under load steps are mixtures that seldom repeat, the device is the bound, and a
        # capture costs more than its replays save (measured: 64 streams at 8B sizes ran 12 %
        # longer with every repeated mixture captured).
        self._graphs: Dict[tuple, "_StepGraph"] = {}       # (batch size | shape, key of the step's ``after``)
        self._shape_seen: Dict[tuple, int] = {}
        self._shape_order: List[tuple] = []
        self.max_shape_graphs = 4
        self.shape_graph_entries = 1
        self.shape_graphs = True
        self.after_result = None
        self._capture_stream = None
        self.cuda_graphs = (cuda_graphs and ops is None and self.rt.device.type == "cuda"
                            and all(getattr(p, "graph_safe", False)
                                    for p in self.model._owners().values()))
        self.graph_replays = 0

    @property
    def vocab_size(self) -> int:
        return self.spec.head.vocab_size

    # ---------------------------------------------------------------- requests
    def open(self, request: Hashable) -> bool:
        """Admit ``request`` (a slot for its block-table row and state); False if none is free."""
        return self.cache.open(request) is not None

    def close(self, request: Hashable) -> None:
        """The request is finished: what it holds is given back."""
        self.cache.close(request)

    # -------------------------------------------------------------------- step
    def step(self, entries: Sequence[StepEntry], feed=None, after=None) -> torch.Tensor:
        """Run the entries' tokens as one batch from the cache; returns the logits at the wanted
        places, float32 [wanted, vocab] on the device, in the order of the entries.  (After a step
        of single tokens, all wanted, they are the captured graph's own rows: the next such step of
        the same batch size writes over them, so keep a copy if you need them longer.)

        ``after``: a callable run on the logits right behind the model (sampling on the device);
        what it returns is kept in ``after_result``.  In a decode step that is replayed from a
        captured graph it is part of the graph, so it has to launch the same work on arrays at the
        same addresses every time it is called for a batch size; ``after.key`` names it (a graph
        is kept per batch size and key).

        ``feed = (source, places, which)`` says that some tokens of this step are on the device
        already (the previous step sampled them there and the host has not read them yet): entry
        ``which[i]`` brings one token, whose value in ``entries`` is ignored; it is
        ``source[places[i]]`` (``source``: int32 on the device)."""
        cache = self.cache
        if feed is not None:
            source, places, which = feed
            if len(places) != len(which) or any(len(entries[k].tokens) != 1 for k in which) \
                    or any(not 0 <= p < source.numel() for p in places):
                raise ValueError("feed: one place in the source per entry, and entries of one token")
        starts = [cache.length(e.request) for e in entries]
        seen = set()
        for e in entries:
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
        V = self.spec.embedding.vocab_size
        # (a prompt portion comes as a list of thousands of Python ints: turned into an array once,
        # checked and later packed as an array)
        tokens = [_token_array(e.tokens) for e in entries]
        for e, a in zip(entries, tokens):
            if a is None or (a.size and not (0 <= int(a.min()) and int(a.max()) < V)):
                raise ValueError(f"request {e.request!r}: token id outside [0, {V})")
        # pages for the whole step or for none of it: lengths first, then the pools' room for all
        # entries together (every group hands out the same number of pages), then the reservations
        for e, s in zip(entries, starts):
            if s + len(e.tokens) > self.max_model_len:
                raise OutOfPages(f"request {e.request!r}: {s + len(e.tokens)} tokens exceed the "
                                 f"engine's max_model_len {self.max_model_len}")
        need = [cache.pages_needed(e.request, s + len(e.tokens)) for e, s in zip(entries, starts)]
        if sum(need) > cache.free_pages():
            short = next(e for e, n in zip(entries, need) if n)
            raise OutOfPages(
                f"the step needs {sum(need)} more pages (request {short.request!r}: "
                f"{cache.pages_needed(short.request, cache.length(short.request) + len(short.tokens))}), "
                f"{cache.free_pages()} are free")
        for e, s in zip(entries, starts):
            if not cache.reserve(e.request, s + len(e.tokens)):
                raise OutOfPages(f"request {e.request!r}: no pages left")     # not reached: checked above
        moves: List[np.ndarray] = []
        if feed is not None:
            lens = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=len(entries))
            first = np.concatenate(([0], np.cumsum(lens[:-1]))).astype(np.int32)   # entry -> its first token
            moves = [first[np.asarray(which, dtype=np.int64)], np.asarray(places, dtype=np.int32)]
        key = self._graph_key(entries, tokens, after) if self.cuda_graphs else None
        if key is not None:
            logits = self._step_with_graph(key, entries, starts, moves, None if feed is None else source,
                                           tokens, after)
            n_tokens = sum(len(t) for t in tokens)
        else:
            ctx, dev_moves = self.prepare_context(entries, starts, moves, tokens)
            if feed is not None:
                self.rt.ops.move_i32(ctx.token_ids, dev_moves[0], source, dev_moves[1])
            logits, n_tokens = self.model.forward(ctx, cache), ctx.n_tokens
            self.after_result = after(logits) if after is not None and logits.shape[0] else None
        for e, s in zip(entries, starts):
            cache.commit(e.request, s + len(e.tokens))
        self.steps += 1
        self.tokens_run += n_tokens
        return logits

    # ------------------------------------------------------------ decode graphs
    def _graph_key(self, entries: Sequence[StepEntry], tokens: Sequence[np.ndarray], after) -> Optional[tuple]:
        """The key of the graph this step replays (or is about to be captured into), or None for a
        step that is launched kernel by kernel."""
        after_key = getattr(after, "key", None) if after is not None else None
        if all(len(t) == 1 and list(e.want) == [0] for e, t in zip(entries, tokens)):
            return (len(entries), after_key)
        if not self.shape_graphs or len(entries) > self.shape_graph_entries:
            return None
        key = (tuple(len(t) for t in tokens), tuple(tuple(e.want) for e in entries), after_key)
        if key in self._graphs:
            self._shape_order.remove(key)
            self._shape_order.append(key)
            return key
        if len(self._shape_seen) > 4096:
            self._shape_seen.clear()
        seen = self._shape_seen[key] = self._shape_seen.get(key, 0) + 1
        if seen < 2:
            return None
        del self._shape_seen[key]
        if key in self._shape_order:                 # promoted before, never captured (its step failed)
            self._shape_order.remove(key)
        while len(self._shape_order) >= self.max_shape_graphs:      # the least recently used goes
            self._graphs.pop(self._shape_order.pop(0), None)
        self._shape_order.append(key)
        return key

    def _step_with_graph(self, key: tuple, entries: Sequence[StepEntry], starts: Sequence[int],
                         moves: List[np.ndarray], source: Optional[torch.Tensor],
                         tokens: Sequence[np.ndarray], after=None) -> torch.Tensor:
        """A step whose shape has a graph: single decode tokens, all wanted (one graph a batch
        size), or a shape with prompt portions that keeps coming.  The step's metadata and the
        block-table cells that changed are copied into buffers at fixed addresses first;
        everything else happens inside the graph (run once without capture, then captured, then
        replayed).  The logits of a decode step live in the graph's own memory and are overwritten
        by the next step of the same batch size; those of a step with prompt portions are copied
        out."""
        cache, R = self.cache, len(entries)
        st = self._graphs.get(key)
        if st is None:
            st = self._graphs[key] = _StepGraph(R, sum(len(t) for t in tokens), sum(len(e.want) for e in entries),
                                                len(cache.groups), self.page_size, self.rt.device)
        extra: List[np.ndarray] = []
        for gi in range(len(cache.groups)):
            cells, values = cache.take_update_arrays(gi)
            if len(cells) > st.cap:                      # rare (many requests closed): plain path
                idx = torch.from_numpy(cells[st.cap:].copy()).to(self.rt.device)
                val = torch.from_numpy(values[st.cap:].copy()).to(self.rt.device)
                self.rt.ops.scatter_i32(cache.groups[gi].dev_table, idx, val)
                cells, values = cells[:st.cap], values[:st.cap]
            packed = np.zeros(1 + 2 * st.cap, dtype=np.int32)
            packed[0] = len(cells)
            packed[1:1 + len(cells)] = cells
            packed[1 + st.cap:1 + st.cap + len(cells)] = values
            extra.append(packed)
        ctx, dev_extra = self._ctx.build(
            tokens, list(starts), [cache.slot(e.request) for e in entries],
            [e.want for e in entries], extra + moves, static=st.meta)
        ctx.fixed_launch = True
        if moves:                                    # after the metadata copy, before the graph
            self.rt.ops.move_i32(ctx.token_ids, dev_extra[-2], source, dev_extra[-1])

        def run():
            for gi, g in enumerate(cache.groups):
                self.rt.ops.scatter_i32_counted(g.dev_table, dev_extra[gi], st.cap)
            logits = self.model.forward(ctx, cache)
            st.after_result = after(logits) if after is not None and logits.shape[0] else None
            return logits

        if st.graph is None:
            if st.warm < 1:                              # once eagerly: loads libraries, sizes scratch
                st.warm += 1
                logits = run()
                self.after_result = st.after_result
                return logits
            torch.cuda.synchronize(self.rt.device)
            graph = torch.cuda.CUDAGraph()
            try:
                # Captured by hand on a side stream: the context manager of the library would also
                # collect garbage and hand all cached device memory back before every capture, which
                # costs tens of milliseconds each time a new batch size turns up in a serving run.
                main = torch.cuda.current_stream(self.rt.device)
                side = self._capture_stream
                if side is None:
                    side = self._capture_stream = torch.cuda.Stream(self.rt.device)
                side.wait_stream(main)
                # No cyclic garbage collection while the stream captures: collecting an engine
                # that is no longer used (its graphs, streams and events) makes calls that a
                # capture does not survive, at whatever moment the collector happens to run.
                collecting = gc.isenabled()
                gc.disable()
                try:
                    with torch.cuda.stream(side):
                        graph.capture_begin()
                        try:
                            st.logits = run()
                        finally:
                            graph.capture_end()
                finally:
                    if collecting:
                        gc.enable()
                main.wait_stream(side)
            except RuntimeError as e:
                # these launches could not be captured: such steps go kernel by kernel from now on
                # (a shape with prompt portions that fails leaves the decode graphs alone)
                import warnings
                if len(key) == 3:
                    warnings.warn(f"CUDA graph capture failed ({e}); steps with prompt portions run without graphs")
                    self.shape_graphs = False
                    for k in self._shape_order:
                        self._graphs.pop(k, None)
                    self._shape_order.clear()
                else:
                    warnings.warn(f"CUDA graph capture failed ({e}); decode steps run without graphs")
                    self.cuda_graphs = False
                torch.cuda.synchronize(self.rt.device)
                logits = run()
                self.after_result = st.after_result
                return logits
            st.graph = graph
            # the capture did not execute anything: the replay below runs this step
        st.graph.replay()
        self.graph_replays += 1
        self.after_result = st.after_result
        if len(key) == 3:
            # a shape with prompt portions: the caller gets rows of its own (who asks for the logits
            # of prompt positions tends to keep them); decode steps hand out the graph's rows
            return st.logits.clone()
        return st.logits

    def check_kernels(self) -> None:
        """Raise if a kernel recorded a fault (a page not held, a token outside the table).
        Synchronises the device."""
        check = getattr(self.rt.ops, "check_status", None)
        if check is not None:
            check()

    def prepare_context(self, entries: Sequence[StepEntry], starts: Sequence[int],
                        more: Sequence[np.ndarray] = (), tokens: Optional[Sequence[np.ndarray]] = None):
        """Build the step's device metadata and bring the device block tables up to date.
        Returns the context and the int32 arrays of ``more`` on the device (they ride along in
        the metadata's one copy)."""
        cache = self.cache
        extra: List[np.ndarray] = []
        for gi in range(len(cache.groups)):
            extra.extend(cache.take_update_arrays(gi))        # later writes to one cell win
        if tokens is None:
            tokens = [e.tokens for e in entries]
        ctx, dev_extra = self._ctx.build(
            tokens, list(starts),
            [cache.slot(e.request) for e in entries], [e.want for e in entries], extra + list(more))
        for gi, g in enumerate(cache.groups):
            idx, val = dev_extra[2 * gi], dev_extra[2 * gi + 1]
            if idx.numel():
                self.rt.ops.scatter_i32(g.dev_table, idx, val)
        return ctx, dev_extra[2 * len(cache.groups):]
