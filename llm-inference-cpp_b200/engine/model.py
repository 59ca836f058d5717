"""The model as the engine sees it: parts in their run order, and one step function.

``step`` is the successor of the reference's ``forward_cached``
(src/model/transformer.cpp:192-306): it runs only the tokens it is given, from the
cache that earlier steps left, and returns logits at the wanted places only — the
final norm and the head run on those rows alone (the reference normalises all rows
and multiplies the last, :298-305).  Unlike the reference it takes a batch of
sequences with unequal lengths in one call.
"""
from __future__ import annotations

import torch

from ..cache.storage import CacheBinding, KVRequest, SequenceCache, StateRequest
from ..parts.build import build_parts, expected_tensors
from ..parts.spec import ModelSpec
from .batch import SequenceStep, StepBuffers, plan_step
from ..ops import kernels
from .runtime import Runtime


class Model:
    def __init__(self, spec: ModelSpec, tensors: dict, dtype: torch.dtype, device="cuda:0", config=None):
        self.spec = spec
        self.config = config
        self.rt = Runtime(dtype, device)
        self.embedding, self.layers, self.final_norm, self.head = build_parts(spec, tensors, self.rt)
        for call in spec.schedule:
            if not (0 <= call.layer < len(self.layers)):
                raise ValueError(f"schedule names layer {call.layer}, but the model has {len(self.layers)}")
        for i, call in enumerate(spec.schedule):
            if call.cache_of is not None and not (0 <= call.cache_of < len(spec.schedule)):
                raise ValueError(f"schedule call {i} reads the cache of call {call.cache_of}, which does not exist")
        self.buffers = StepBuffers(self.rt.device, self.rt)
        self._graphs = None
        self._prompt_graphs = None
        self._ids_host = None        # pinned: the chosen ids come to the host through it
        # Short prompt steps are padded to a shape and replayed from recorded graphs (engine/graphs.py) where every
        # part says that rows of no sequence do it no harm (``takes_padding_rows``), in the compute type that serving uses.
        parts = [self.embedding, self.final_norm, self.head]
        for layer in self.layers:
            parts += [layer.block, *layer.parts.values()]
        self.pads_prompts = dtype == torch.bfloat16 and all(getattr(p, "takes_padding_rows", False) for p in parts)
        self.last_logits = None      # fp32 [rows, vocab] of the latest step_and_choose (scratch: valid until the next step)
        self.parameter_count = sum(int(torch.tensor(d.shape).prod()) for d in expected_tensors(spec).values())

    # -- sizes -----------------------------------------------------------------------------
    @property
    def dtype(self):
        return self.rt.dtype

    @property
    def device(self):
        return self.rt.device

    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    def weight_bytes(self) -> int:
        """Bytes of every weight a step reads once (a tied table counts once)."""
        total = self.embedding.weight_bytes() + self.head.weight_bytes()
        used = {call.layer for call in self.spec.schedule}
        for i in used:
            for p in self.layers[i].parts.values():
                total += p.weight_bytes() if hasattr(p, "weight_bytes") else 0
        return total

    # -- cache -----------------------------------------------------------------------------
    def new_cache(self, max_tokens: int, n_slots: int | None = None) -> SequenceCache:
        """A cache for at most ``max_tokens`` live tokens (each sequence rounded up to whole pages).

        Scheduled calls with equal cache requests share a group; a call that reads another
        call's cache gets that call's place in the group and writes nothing.
        """
        requests = [self.layers[c.layer].mixer.cache_request() for c in self.spec.schedule]
        kv_groups: dict = {}
        state_groups: dict = {}
        place = []
        for i, (call, req) in enumerate(zip(self.spec.schedule, requests)):
            if call.cache_of is not None:
                place.append(None)
                continue
            table = kv_groups if isinstance(req, KVRequest) else state_groups if isinstance(req, StateRequest) else None
            if table is None:
                place.append(("none", None, 0))
                continue
            table.setdefault(req, [])
            place.append(("kv" if table is kv_groups else "state", req, len(table[req])))
            table[req].append(i)
        cache = SequenceCache([(r, len(c)) for r, c in kv_groups.items()],
                              [(r, len(c)) for r, c in state_groups.items()],
                              max_tokens, self.spec.max_positions, self.rt.dtype, self.rt.device, n_slots=n_slots)
        kv_index = {r: g for r, g in zip(kv_groups, cache.kv_groups)}
        st_index = {r: g for r, g in zip(state_groups, cache.state_groups)}
        bindings = []
        for i, call in enumerate(self.spec.schedule):
            src = place[i] if call.cache_of is None else place[call.cache_of]
            if src is None:
                raise ValueError(f"schedule call {i} reads the cache of call {call.cache_of}, which has none of its own")
            kind, req, idx = src
            if call.cache_of is not None and requests[i] != req:
                raise ValueError(f"schedule call {i} cannot read the cache of call {call.cache_of}: their needs differ")
            group = kv_index[req] if kind == "kv" else st_index[req] if kind == "state" else None
            bindings.append(CacheBinding(group, idx, writes=call.cache_of is None))
        cache.bindings = bindings
        cache.owner = self
        # the (mixer, binding) pairs whose launches may depend on more than a step's padded shape, one of a kind
        planners = {}
        for call, binding in zip(self.spec.schedule, bindings):
            mixer = self.layers[call.layer].mixer
            if hasattr(mixer, "step_plan"):
                planners.setdefault((id(binding.group), mixer.cache_request(), getattr(mixer, "n_heads", None)),
                                    (mixer, binding))
        cache.planners = list(planners.values())
        return cache

    def step_plan_token(self, ctx, cache) -> tuple:
        """What a recorded step depends on beside its padded shape: the mixers' own plans for this step (a decode
        kernel's split follows the live sequences)."""
        token = getattr(ctx, "plan_token", None)      # a context that is continued keeps its sizes, so its token too
        if token is None:
            token = ctx.plan_token = tuple(m.step_plan(ctx, b) for m, b in getattr(cache, "planners", ()))
        return token

    # -- the step --------------------------------------------------------------------------
    def step(self, cache: SequenceCache, seqs, pad_seqs_to: int = 0, pad_pages_to: int = 0,
             trace: list | None = None) -> torch.Tensor:
        """Run the given tokens of the given sequences; fp32 logits ``[wanted, vocab]`` in entry order.

        ``seqs``: :class:`SequenceStep` items (slot, next tokens, wanted places).  The returned
        tensor is scratch: it is valid until the next step.
        """
        if getattr(cache, "owner", None) is not self:
            raise ValueError("step: cache was not created by this model")
        if (self.pads_prompts and trace is None and not pad_seqs_to and not pad_pages_to and seqs
                and max(len(s.tokens) for s in seqs) > 1):
            from . import graphs
            if graphs.RECORD:
                if self._prompt_graphs is None:
                    self._prompt_graphs = graphs.PromptGraphs(self)
                logits = self._prompt_graphs.step(cache, seqs)
                if logits is not None:
                    return logits
        ctx = plan_step(cache, seqs, self.spec.vocab_size, self.buffers, pad_seqs_to, pad_pages_to)
        self._last_h2d = ctx.h2d_bytes
        return self.run(ctx, cache, trace)

    def run(self, ctx, cache, trace: list | None = None) -> torch.Tensor:
        """The device work of a step for an uploaded context (what a recorded graph replays).

        ``trace``, when given, receives copies of the residual stream after the embedding and
        after every scheduled call, and the final norm of all rows — the states of the
        reference's ForwardTrace (include/llmi/model/transformer.hpp:14-19).
        """
        x = self.embedding.forward(ctx.token_ids, ctx)
        if trace is not None:
            trace.append(x.clone())
        # A block may hand the next one its first norm half done (norm deferral, see parts/block.py): `entry`
        # is that norm's deferred form, filled by the block before; blocks without the extras run as ever.
        blocks = [self.layers[call.layer].block for call in self.spec.schedule]
        entry = None
        for i, (block, binding) in enumerate(zip(blocks, cache.bindings)):
            if hasattr(block, "entry_norm"):
                nxt = getattr(blocks[i + 1], "entry_norm", None) if i + 1 < len(blocks) else None
                entry = block.forward(x, ctx, binding, entry=entry, next_norm=nxt)
            else:
                block.forward(x, ctx, binding)
                entry = None
            if trace is not None:
                trace.append(x.clone())
        if trace is not None:
            trace.append(self.final_norm.forward(x, scratch_name="trace_norm_out").float().clone())
        if ctx.n_want == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.rt.device)
        h = self.final_norm.forward(x, rows=ctx.want_rows, scratch_name="final_norm_out")
        return self.head.forward(h)

    def step_and_choose(self, cache, seqs, sampler, streams=None, use_graphs: bool = True):
        """One step followed by the choice of one token per wanted row; returns the ids on the host.
        The logits the choice was made from stay in ``last_logits`` until the next step."""
        if use_graphs and all(len(s.tokens) == 1 for s in seqs) and all(s.want == [0] for s in seqs):
            if self._graphs is None:
                from .graphs import DecodeGraphs
                self._graphs = DecodeGraphs(self)
            return self._ids_to_host(self._graphs.step(cache, seqs, sampler, streams))
        logits = self.step(cache, seqs)
        self.last_logits = logits
        ids = sampler.choose(logits, streams)
        return self._ids_to_host(ids)

    def _ids_to_host(self, ids: torch.Tensor) -> torch.Tensor:
        """Device int32 ids -> a host tensor of their own: one copy into pinned memory and the wait for it in one
        library call (a tensor's own way to the host costs about 20 us more after the step is done)."""
        n = ids.numel()
        if n == 0 or ids.dtype != torch.int32 or not ids.is_contiguous():
            return ids.cpu()
        if self._ids_host is None or self._ids_host.numel() < n:
            self._ids_host = torch.empty(max(256, 2 * n), dtype=torch.int32, pin_memory=True)
        kernels.copy_to_host(self._ids_host.data_ptr(), ids.data_ptr(), 4 * n)
        return self._ids_host[:n].clone()

    @property
    def last_h2d_bytes(self) -> int:
        return getattr(self, "_last_h2d", 0)
