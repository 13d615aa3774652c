"""The step function: one batch of (request, its next tokens) through the model.

``ModelRunner`` owns the bound model, the cache manager and the step packer.  ``step``
takes any mix of prompt portions and single decode tokens, runs exactly the tokens it is
given as one batch against the cache that earlier steps left, writes their keys, values and
states, and returns float32 logits at the wanted places.  It is the only forward pass of the
package: generation, the scheduler, trace replay and the benchmark all go through it.

It corresponds to the reference's ``ExecutionBackend::forward`` over
``PagedLfm2::prepare`` + ``forward_prepared``
(crates/vapi-engine/src/backend.rs:303-336, crates/vapi-backend-candle/src/models/lfm2.rs:718-818).
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Optional, Sequence

import torch

from .. import ops
from ..cache.manager import CacheManager
from ..config.model import eos_token_ids, load_config_json, resolve_architecture
from ..models.plan import ModelPlan
from ..parts.base import CacheView
from ..weights.loader import load_tensors
from ..weights.random import random_tensors
from .step import StepContext, StepEntry, StepPacker, validate_step

DTYPES = {"float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
          "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype {name} is not supported (float32, bfloat16)")
        return name
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype `{name}` is not one of {sorted(DTYPES)}")


class ModelRunner:
    #: tokens per cache page (the reference's block is 32 tokens, crates/vapi-core/src/config.rs:15;
    #: 64 keeps a page of one kv head at 8 KB for head_dim 64 in bfloat16)
    default_page_size = 64

    def __init__(self, plan: ModelPlan, tensors: Dict[str, torch.Tensor], *, dtype, device="cuda",
                 page_size: int = default_page_size, num_pages: Optional[int] = None, max_requests: int = 64,
                 max_batched_tokens: int = 8192, max_context: Optional[int] = None,
                 watermark: float = 0.0, kv_cache_fraction: float = 0.85, validate: bool = True):
        self.plan, self.dtype, self.device = plan, parse_dtype(dtype), torch.device(device)
        if self.device.type == "cuda":
            ops.strict_fp32()
        plan.bind(tensors, self.dtype)
        self.vocab_size = plan.vocab_size
        self.max_context = min(int(max_context or plan.max_positions), plan.max_positions)
        self.max_batched_tokens = int(max_batched_tokens)
        # checking every batch on the host is a debugging aid (the reference does it in debug
        # builds, crates/vapi-backend-candle/src/backend.rs:486-487); VAPI_VALIDATE=1 forces it
        self.validate = bool(validate) or os.environ.get("VAPI_VALIDATE") == "1"
        sites = plan.cache_sites()
        if num_pages is None:
            num_pages = self._pages_from_memory(sites, page_size, max_requests, kv_cache_fraction)
        self.cache = CacheManager(sites, page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                                  dtype=self.dtype, device=self.device, watermark=watermark)
        width = -(-self.max_context // page_size)
        width = -(-width // 4) * 4
        self.packer = StepPacker(self.cache, self.device, self.max_batched_tokens,
                                 max(max_requests, 1) , width)
        # The kernels' status word and the sampled tokens share one buffer, word first, so that the
        # word travels to the host in the same copy as a step's tokens.
        self.status_and_sampled = torch.zeros(1 + max(256, max_requests), dtype=torch.int32, device=self.device)
        #: non-zero once a kernel refused an index or gave up a bounded wait (see :data:`STATUS_NAMES`)
        self.status = self.status_and_sampled[:1]
        #: the tokens the last step sampled on the device, one per wanted row.  A step that is
        #: enqueued before the host has read them takes its input tokens from here.
        self.sampled = self.status_and_sampled[1:]
        # one CacheView skeleton per run-order entry
        self._site_of: List[Optional[int]] = []
        for i, call in enumerate(plan.order):
            owner = call.cache_of if call.cache_of is not None else i
            self._site_of.append(owner if self.cache.site_tensor(owner) is not None else None)
        self._site_buffers = {s: self.cache.site_buffers(s) for s in set(self._site_of) if s is not None}
        self.steps_run = 0
        self.graph_max_batch = min(64, max_requests)
        self._graphs: Dict[int, Any] = {}
        self._graphs_off = self.device.type != "cuda"

    # ---- construction -------------------------------------------------------------
    @classmethod
    def from_dir(cls, model_dir: str, *, dtype="bfloat16", device="cuda", **kw) -> "ModelRunner":
        """Load a model folder (config.json + safetensors); the architecture is chosen by
        config.json through the registry."""
        cfg_json = load_config_json(model_dir)
        arch = resolve_architecture(cfg_json)
        plan = arch.plan(arch.parse(cfg_json))
        eos = eos_token_ids(model_dir, cfg_json)
        if eos:
            plan.eos_token_ids = eos
        tensors = load_tensors(model_dir, plan.tensor_specs(), parse_dtype(dtype), device)
        return cls(plan, tensors, dtype=dtype, device=device, **kw)

    @classmethod
    def from_random(cls, config_json: Dict[str, Any], seed: int, *, dtype="bfloat16", device="cuda",
                    std: float = 0.02, norm_init: str = "ones", **kw) -> "ModelRunner":
        """Random weights drawn directly on the device, without a folder in between."""
        arch = resolve_architecture(config_json)
        plan = arch.plan(arch.parse(config_json))
        dt = parse_dtype(dtype)
        raw = random_tensors(plan, seed, std, norm_init, torch.float32, device=str(device))
        specs = {s.name: s for s in plan.tensor_specs()}
        tensors = {k: (v if specs[k].role != "matrix" else v.to(dt)) for k, v in raw.items()}
        return cls(plan, tensors, dtype=dtype, device=device, **kw)

    def _pages_from_memory(self, sites, page_size, max_requests, fraction) -> int:
        """free memory x fraction / bytes per page, the reference's sizing rule
        (crates/vapi-backend-candle/src/backend.rs:385-400) with the state slots taken off first."""
        from ..parts.base import PagedSpec, StateSpec
        esize = 4 if self.dtype == torch.float32 else 2
        per_token = sum(s.elems_per_token() for _, s in sites if isinstance(s, PagedSpec)) * esize
        per_req = 0
        for _, s in sites:
            if isinstance(s, StateSpec):
                k = 1
                for d in s.shape:
                    k *= d
                per_req += k * esize
        if self.device.type != "cuda":
            raise ValueError("num_pages must be given when the device is not CUDA")
        free, _ = torch.cuda.mem_get_info(self.device)
        budget = int(free * fraction) - per_req * (max_requests + 1)
        pages = budget // max(per_token * page_size, 1) if per_token else max_requests
        # never more than every request at full context could use
        cap = max_requests * -(-self.max_context // page_size)
        pages = min(int(pages), cap)
        if pages <= 0:
            raise ValueError("the cache budget leaves no room for a single page")
        return pages

    # ---- the step ------------------------------------------------------------------
    def views(self, ctx: StepContext) -> List[CacheView]:
        out = []
        for i, call in enumerate(self.plan.order):
            site = self._site_of[i]
            if site is None:
                out.append(CacheView("none"))
                continue
            kind, gi = self.cache.site_kind(site)
            out.append(CacheView(kind, self.cache.site_tensor(site),
                                 ctx.groups[gi] if kind == "paged" else None,
                                 write=call.cache_of is None,
                                 buffers=self._site_buffers[site] if kind == "paged" else None,
                                 spec=self.cache.site_spec(site)))
        return out

    def forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """Device work of a step for a prepared context; returns float32 logits [rows, vocab]
        or None when no logits are wanted (the caches are written either way)."""
        if self.device.type == "cuda":
            with ops.one_stream():
                return self._forward(ctx)
        return self._forward(ctx)

    def _forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        plan = self.plan
        if ctx.unknown_tokens:
            ops.resolve_tokens(ctx.tokens, ctx.token_src, self.sampled, self.status)
        for pe in plan.position_encodings:
            ctx.pos[pe.name] = pe.prepare(ctx)
        views = self.views(ctx)
        ctx.fused = (self.device.type == "cuda" and self.dtype == torch.bfloat16 and ops.use_skinny
                     and (ctx.n <= (ops.TC_MAX_ROWS if ops.use_tc else ops.SKINNY_MAX_ROWS)
                          or 0 < ops.PROMPT_MIN_ROWS <= ctx.n))
        if ctx.fused:
            return self._forward_few_rows(ctx, views)
        x = plan.embedding.forward(ctx)
        delta = None
        for i, call in enumerate(plan.order):
            delta = plan.layers[call.layer].forward(x, delta, ctx, views[i])
        if ctx.logits_rows is None:
            return None
        xn = plan.final_norm.apply(x, delta, ctx.dtype, rows=ctx.logits_rows)
        return plan.head.forward(xn)

    def _forward_few_rows(self, ctx: StepContext, views: List[CacheView]) -> Optional[torch.Tensor]:
        """The same model for a step of at most 16 rows (decode): every block runs in its
        stream form, see :meth:`PreNormBlock.forward_stream`."""
        from ..parts.base import StreamState
        plan = self.plan
        order = plan.order

        def reader_weight(i: int):
            """Weight of the norm that reads the stream before run-order entry i (or the final norm)."""
            if i >= len(order):
                return plan.final_norm.stream_weight()
            blk = plan.layers[order[i].layer]
            return blk.first_norm().stream_weight() if hasattr(blk, "first_norm") else None

        w0 = reader_weight(0)
        if w0 is not None:
            x, ss, xw = plan.embedding.forward(ctx, w0)
            state = StreamState(xw, ss)
        else:
            x, state = plan.embedding.forward(ctx), None
        for i, call in enumerate(order):
            blk = plan.layers[call.layer]
            nw = reader_weight(i + 1)
            if hasattr(blk, "forward_stream"):
                state = blk.forward_stream(x, state, ctx, views[i], nw)
            else:
                delta = blk.forward(x, None, ctx, views[i])
                if nw is None:
                    ops.add_residual(x, delta)
                    state = None
                else:
                    state = StreamState(*reversed(ops.add_residual_ss(x, delta, nw)))
        if ctx.logits_rows is None:
            return None
        if ctx.rows_identity and state is not None:
            a = plan.final_norm.deferred(state)
            if a is not None:
                logits = plan.head.forward_stream(a)
                if logits is not NotImplemented:
                    return logits
        xn = plan.final_norm.apply(x, None, ctx.dtype, rows=ctx.logits_rows)
        return plan.head.forward(xn)

    def step(self, entries: Optional[Sequence[StepEntry]], plan=None) -> Optional[torch.Tensor]:
        """Run one batch.  Pages must have been reserved by the caller
        (``cache.reserve(rc, rc.num_tokens + len(tokens))``): what happens when they run out
        is the scheduler's decision, not the step function's.  ``plan``, instead of ``entries``,
        is a step that the scheduler has planned: the host runtime then packs it straight from
        its own arrays."""
        if self.validate:
            validate_step(plan.entries if plan is not None else entries, self.cache, self.vocab_size,
                          self.max_context)
        ctx = self.packer.pack(entries, self.dtype, status=self.status, plan=plan)
        logits = self.forward(ctx)
        self._commit(entries, plan)
        self.steps_run += 1
        return logits

    def _commit(self, entries, plan) -> None:
        if plan is not None:
            plan.commit_cache()
        else:
            for e in entries:
                self.cache.commit(e.cache, e.start + len(e.tokens))

    # ---- captured decode steps --------------------------------------------------------
    def _bucket(self, S: int) -> int:
        """The fixed shape a decode step of S sequences is padded to: the next power of two, but
        never more than the packer and the scratch buffers were sized for."""
        b = 1
        while b < S:
            b *= 2
        return min(b, self.graph_max_batch)

    def _capture(self, B: int):
        """Capture the device work of a pure decode step of B sequences into a CUDA graph
        (the reference does the same per power-of-two bucket up to 64,
        crates/vapi-backend-candle/src/backend.rs:1015-1019, 1124-1214).  Inputs live at fixed
        offsets of the packer's device buffer; padding rows use pages and a state slot that
        no request owns."""
        if self.packer._pad_pages is None:
            pages = self.cache.set_aside_pages()
            if pages is None:
                raise RuntimeError("no page can be set aside for the padding rows")
            self.packer.set_pad_pages(pages)
        width = self.packer.max_width
        ctx = self.packer.pack([], self.dtype, n_cap=B, s_cap=B, width=width, status=self.status)
        ctx.max_k = self.max_context
        ctx.unknown_tokens = True       # the captured step always looks: token_src says where
        for gi, splits in enumerate(self._decode_splits(B)):
            ctx.groups[gi].splits, ctx.groups[gi].max_k = splits, self.max_context
        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(2):
                ctx.pos = {}
                self.forward(ctx)
        cur.wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        ctx.pos = {}
        before = ops.launch_count
        # The collector must not run inside the capture: if it frees another runner's graphs there
        # (objects in reference cycles die whenever it happens to run), releasing their memory is an
        # operation that a capturing stream does not permit, and this capture is lost with it.
        import gc
        gc.collect()
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph):
                logits = self.forward(ctx)
        finally:
            if was_enabled:
                gc.enable()
        return graph, logits, ops.launch_count - before

    def _decode_splits(self, B: int) -> List[int]:
        """Per paged cache group: into how many slices a captured decode step of B sequences cuts
        a sequence's keys, the most that any mixer of the group asks for."""
        best = [1] * len(self.cache.paged)
        for i, call in enumerate(self.plan.order):
            site = self._site_of[i]
            if site is None:
                continue
            kind, gi = self.cache.site_kind(site)
            mixer = getattr(self.plan.layers[call.layer], "mixer", None)
            if kind == "paged" and mixer is not None:
                best[gi] = max(best[gi], int(mixer.decode_splits(B, self.max_context, self.cache.page_size, self.dtype)))
        return best

    def step_decode_graph(self, entries: Optional[Sequence[StepEntry]], plan=None) -> Optional[torch.Tensor]:
        """A pure decode step (one token and one wanted row per request) through a captured
        graph; None when the step is not of that shape or graphs are unavailable, in which
        case the caller uses :meth:`step`."""
        S = plan.num_entries if plan is not None else len(entries)
        if self._graphs_off or S == 0 or S > self.graph_max_batch:
            return None
        if plan is not None:
            if not plan.pure_decode:
                return None
        else:
            for e in entries:
                if len(e.tokens) != 1 or list(e.want) != [0]:
                    return None
        if self.validate:
            validate_step(plan.entries if plan is not None else entries, self.cache, self.vocab_size,
                          self.max_context)
        B = self._bucket(S)
        if B not in self._graphs:
            if self.packer._pad_pages is None and self.cache.paged:
                pages = self.cache.set_aside_pages()
                if pages is None:         # no page to spare for padding rows: no bucket can be captured
                    self._graphs_off = True
                    return None
                self.packer.set_pad_pages(pages)
            try:
                self._graphs[B] = self._capture(B)
            except Exception as exc:      # this bucket decodes eagerly; the others keep their graphs
                import warnings
                warnings.warn(f"CUDA graph capture of a decode step of {B} sequences failed ({exc}); "
                              f"steps of that size run eagerly")
                self._graphs[B] = None
                if self.device.type == "cuda":
                    torch.cuda.synchronize()
        if self._graphs[B] is None:
            return None
        graph, logits, kernels = self._graphs[B]
        self.packer.pack(entries, self.dtype, n_cap=B, s_cap=B, width=self.packer.max_width, status=self.status,
                         plan=plan)
        graph.replay()
        ops.launch_count += kernels
        self._commit(entries, plan)
        self.steps_run += 1
        return logits[:S]

    def check_status(self) -> None:
        """Raise if a kernel met an index it refused to follow (a bad token id, slot or
        page: the host validation should have caught it first) or gave up a bounded wait."""
        self.raise_on_status(int(self.status.item()))

    def raise_on_status(self, code: int) -> None:
        """Turn a status word that was read from the device into a :class:`KernelRefusal` and
        clear the word on the device.  The engine loop calls this with the word that came to the
        host beside a step's sampled tokens, so generation costs no copy or wait of its own."""
        if code:
            self.status.zero_()
            raise KernelRefusal(code)


#: what the kernels write into the status word
STATUS_NAMES = {1: "token id outside the vocabulary", 2: "cache slot outside the pool",
                3: "state slot outside the pool", 4: "page id outside the pool",
                16: "a bounded wait inside a kernel ran out, and the kernel left its output unwritten"}


class KernelRefusal(RuntimeError):
    """A kernel of the step recorded a status: what the step produced cannot be trusted."""

    def __init__(self, code: int):
        self.code = int(code)
        super().__init__(f"a kernel refused to go on: {STATUS_NAMES.get(self.code, f'status {self.code}')}")
