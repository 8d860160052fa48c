"""Model forwards of the serving loop: packed ragged prefill, batched decode (CUDA-graph replay), sampling.

Counterpart of ``astrai/inference/runtime/executor.py:24-421``.  Differences: one packed prefill forward serves
requests of DIFFERENT prompt lengths and different cached-prefix lengths (the reference runs one forward per
``(prompt_len, start_pos)`` group); only the last position of each request goes through the vocabulary projection;
sampling parameters and their host-side facts (largest k, any p < 1, any penalty) are cached per task set so a decode
step performs exactly one device->host transfer (the sampled ids).
"""

from __future__ import annotations

import bisect
import dataclasses

import logging
import time
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
from torch import Tensor

from astrai_b200.inference.cache import PagePool, TaskCacheManager
from astrai_b200.inference.runtime.graph import CudaGraphContext
from astrai_b200.inference.runtime.sample import sample
from astrai_b200.inference.task import Task
from astrai_b200.inference.workspace import InferenceWorkspace

logger = logging.getLogger(__name__)


@contextmanager
def timed(label: str, log: Optional[logging.Logger] = None):
    """CUDA-event timer, active only when the logger is at DEBUG (``ASTR_LOG_LEVEL=DEBUG``)."""
    log = log or logger
    if not log.isEnabledFor(logging.DEBUG):
        yield
        return
    cuda = torch.cuda.is_available()
    if cuda:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
    else:
        tic = time.perf_counter()
    yield
    if cuda:
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
    else:
        ms = (time.perf_counter() - tic) * 1000
    log.debug("%s %.2fms", label, ms)


@dataclass
class SamplingBatchInfo:
    temperatures: Tensor
    top_ks: Tensor
    top_ps: Tensor
    freq_penalties: Tensor
    has_freq: bool
    hints: dict


@dataclass
class DecodeSteadyState:
    task_sig: tuple
    positions: List[int]
    sampling_info: SamplingBatchInfo


def build_sampling_info(tasks: List[Task], device) -> SamplingBatchInfo:
    pin = str(device).startswith("cuda")

    def col(values, dtype):
        return torch.tensor(values, dtype=dtype, pin_memory=pin).to(device, non_blocking=True)

    temps = [t.temperature for t in tasks]
    ks = [t.top_k for t in tasks]
    ps = [t.top_p for t in tasks]
    fs = [t.frequency_penalty for t in tasks]
    hints = {"max_k": max([0] + ks), "top_p_active": any(p < 1.0 for p in ps), "has_freq": any(f != 0 for f in fs),
             "greedy": all(t == 0 for t in temps)}
    return SamplingBatchInfo(col(temps, torch.float32), col(ks, torch.int32), col(ps, torch.float32),
                             col(fs, torch.float32), hints["has_freq"], hints)


def fuse_projection_weights(model) -> int:
    """Lay the q / k / v weights of every GQA layer and the gate / up weights of every dense MLP out as ONE matrix each
    (the separate parameters become views of it), so that a decode step launches one projection GEMM where it launched
    three (or two); stack the routed experts of every MoE layer once for the grouped GEMMs.  The modules pick the fused matrix up through ``fused_qkv`` / ``fused_gate_up``, exactly as under the
    flat-buffer training executors; parameter names, shapes and the state dict are unchanged.  Returns the number of
    fused groups.  Layers with wrapped projections (LoRA) or biases are left alone."""
    fused = 0

    def plain(*mods) -> bool:
        return all(type(m).__name__ == "Linear" and getattr(m, "bias", None) is None and m.weight.dim() == 2 for m in mods)

    for mod in model.modules():
        experts = getattr(mod, "routed_experts", None)
        if experts is not None and getattr(mod, "stacked_experts", 0) is None and len(experts) > 0 and all(
                plain(m.gate, m.up, m.down) for m in experts):
            # mixture of experts: one [E, 2F, D] and one [E, D, F] tensor for the grouped GEMMs instead of a stack per call
            with torch.no_grad():
                w_gu = torch.stack([torch.cat([m.gate.weight.detach(), m.up.weight.detach()], dim=0) for m in experts])
                w_dn = torch.stack([m.down.weight.detach() for m in experts])
                f = experts[0].gate.weight.shape[0]
                for i, m in enumerate(experts):
                    m.gate.weight.data, m.up.weight.data, m.down.weight.data = w_gu[i, :f], w_gu[i, f:], w_dn[i]
                    m.fused_gate_up = w_gu[i]  # the expert's own gate|up matrix is a slice of the stack
            mod.stacked_experts = (w_gu, w_dn)
            fused += 1
            continue
    for mod in model.modules():
        if hasattr(mod, "fused_qkv") and mod.fused_qkv is None and plain(mod.q_proj, mod.k_proj, mod.v_proj):
            parts = [mod.q_proj, mod.k_proj, mod.v_proj]
            attr = "fused_qkv"
        elif hasattr(mod, "fused_gate_up") and mod.fused_gate_up is None and plain(mod.gate, mod.up):
            parts = [mod.gate, mod.up]
            attr = "fused_gate_up"
        else:
            continue
        with torch.no_grad():
            whole = torch.cat([p.weight.detach() for p in parts], dim=0)
            row = 0
            for p in parts:
                n = p.weight.shape[0]
                p.weight.data = whole[row:row + n]
                row += n
        setattr(mod, attr, whole)
        fused += 1
    return fused


class Executor:
    def __init__(self, model, kv_cache: PagePool, task_cache: TaskCacheManager, device=None, dtype=None,
                 enable_cuda_graph: bool = True, max_prefill_tokens: Optional[int] = None, control=None):
        """``control``: a :class:`~astrai_b200.parallel.tp_inference.ReplicatedControl` when several ranks run this executor
        in lockstep on their shares of one model; the first rank's sampled tokens are then used by all."""
        self.model, self.kv_cache, self.task_cache, self.control = model, kv_cache, task_cache, control
        if next(model.parameters()).is_cuda and not model.training:
            fuse_projection_weights(model)
        p = next(model.parameters())
        self.device = torch.device(device) if device is not None else p.device
        self.dtype = dtype or p.dtype
        cfg = self._cfg = getattr(model, "local_config", None) or model.config  # a tensor-parallel rank sizes for its own heads
        head_dim = cfg.hidden_size // cfg.num_attention_heads
        self.max_prefill_tokens = max_prefill_tokens or kv_cache.max_batch_size * kv_cache.max_seq_len
        self._workspace = InferenceWorkspace(kv_cache.max_batch_size, kv_cache.max_seq_len, cfg.num_attention_heads,
                                             head_dim, self.device, self.dtype, n_kv_heads=cfg.num_key_value_heads,
                                             max_prefill_tokens=min(self.max_prefill_tokens, 1 << 20))
        self._decode_cache: Optional[DecodeSteadyState] = None
        self._graph_ctx = CudaGraphContext()
        self._buckets: List[int] = []
        self._graph_supported = (self.device.type == "cuda" and self.dtype == torch.bfloat16
                                 and head_dim in (32, 64, 128, 256) and 1 <= cfg.num_attention_heads // cfg.num_key_value_heads <= 8)
        from astrai_b200.ops import backend as attn_backends

        # decode graphs hold the kernels of the back end that was active at capture: steps under another one run eagerly
        self._graph_backend = attn_backends.get_backend(self.device.type)
        if enable_cuda_graph and self._graph_supported:
            self._graph_ctx.set_enabled(True)
            self._warmup()

    workspace = property(lambda self: self._workspace)

    @property
    def cuda_graph_enabled(self) -> bool:
        return self._graph_ctx.enabled and self._graph_supported

    @staticmethod
    def decode_buckets(b_max: int) -> List[int]:
        """Batch sizes that get a decode graph: 1, 2, 4, every multiple of 8 up to 64, every multiple of 16 above, and
        the maximum.  A step of ``b`` requests replays the graph of the smallest bucket ``>= b`` with the extra rows
        padded (sequence length 0: they read no keys and store nothing), so no graph is ever captured while serving and
        at most a third of the rows of a step are padding (an eighth from 32 requests on)."""
        sizes = {1, 2, 4} | set(range(8, 65, 8)) | set(range(80, b_max + 1, 16)) | {b_max}
        return sorted(x for x in sizes if x <= b_max)

    def _decode_splits(self, rows: int) -> int:
        """KV splits baked into the graph of a bucket: one wave of two CTAs per SM whatever the context length (a graph
        outlives the lengths it was captured with; splits that fall beyond a short sequence return at once)."""
        base = max(rows * self._cfg.num_key_value_heads, 1)
        return max(1, min(148 * 2 // base, self._workspace.decode_o_part.shape[2]))

    def _padded(self, kv, b: int, rows: int):
        """The step's cache view widened to ``rows`` >= ``b`` rows of the workspace (the caller zeroed rows ``b..``)."""
        ws = self._workspace
        return dataclasses.replace(kv, req_pool_indices=ws.req_pool_indices[:rows], seq_lens=ws.seq_lens[:rows],
                                   out_cache_loc=ws.out_cache_loc[:rows], qo_indptr=ws.qo_indptr[: rows + 1],
                                   decode_splits=self._decode_splits(rows))

    def _zero_padding(self, b: int, rows: int):
        ws = self._workspace
        if rows > b:
            for buf in (ws.input_ids, ws.position_ids, ws.seq_lens, ws.req_pool_indices):
                buf[b:rows].zero_()

    def _warmup(self):
        """Capture one decode graph per bucket of :meth:`decode_buckets` (live step, capture, replay)."""
        tc, ws, b_max = self.task_cache, self._workspace, self.kv_cache.max_batch_size
        self._buckets: List[int] = []
        with torch.inference_mode():
            for b in self.decode_buckets(b_max):
                ids = [f"_warmup_{b}_{i}" for i in range(b)]
                if not all(tc.task_alloc(t, [0]) for t in ids):
                    for t in ids:
                        tc.task_free(t)
                    continue
                for step in range(3):  # live, capture, replay
                    for t in ids:
                        tc.task_extend(t, step)
                    kv = self._padded(tc.bind(ids, ws), b, b)
                    ws.put_long(ws.position_ids, [step] * b)
                    tokens = ws.fill_input_ids([0] * b)
                    self._graph_ctx.forward(self.model, key=(b,), input_ids=tokens, kv_cache=kv,
                                            position_ids=ws.position_ids[:b], fwd="decode")
                for t in ids:
                    tc.task_free(t)
                torch.cuda.synchronize()
                if self._graph_ctx.has_graph((b,)):
                    self._buckets.append(b)

    def _bucket(self, b: int) -> int:
        """Smallest captured bucket that holds ``b`` requests (``b`` itself when there is none)."""
        i = bisect.bisect_left(self._buckets, b)
        return self._buckets[i] if i < len(self._buckets) else b

    # -- sampling ---------------------------------------------------------------------------------------------------------
    def _sample(self, logits: Tensor, tasks: List[Task], return_logprobs: bool, info: Optional[SamplingBatchInfo] = None,
                wait: bool = True):
        """Launch the sampler; ``wait=False`` returns a zero-argument callable that reads the tokens back (the one
        device -> host transfer of a step), so the caller can queue more work behind the launch first."""
        info = info or build_sampling_info(tasks, self.device)
        hist = hist_mask = None
        if info.has_freq:
            rows = [t.prompt_ids[-t.rep_window:] + t.output_ids for t in tasks]
            width = max((len(r) for r in rows), default=0)
            hist = torch.zeros(len(tasks), width, dtype=torch.long)
            hist_mask = torch.zeros(len(tasks), width, dtype=torch.bool)
            for i, r in enumerate(rows):
                hist[i, : len(r)] = torch.tensor(r, dtype=torch.long)
                hist_mask[i, : len(r)] = True
            hist, hist_mask = hist.to(self.device), hist_mask.to(self.device)
        out = sample(logits, temperature=info.temperatures, top_k=info.top_ks, top_p=info.top_ps,
                     frequency_penalty=info.freq_penalties, input_ids=hist, input_mask=hist_mask,
                     return_logprobs=return_logprobs, hints=info.hints)
        if self.control is not None:  # one random stream decides for every rank of the replica
            self.control.share_tokens(*(out if return_logprobs else (out,)))

        def finish():
            if not return_logprobs:
                return out.tolist()
            tokens, logp = out
            tokens, logp = tokens.tolist(), logp.tolist()
            for t, lp in zip(tasks, logp):
                t.output_logprobs.append(float(lp))
            return list(zip(tokens, logp))

        return finish() if wait else finish

    # -- prefill ------------------------------------------------------------------------------------------------------------
    def execute_prefill(self, tasks: List[Task], prompt_len: Optional[int] = None, start_pos: Optional[int] = None,
                        return_logprobs: bool = False, end_positions: Optional[Dict[str, int]] = None, wait: bool = True):
        """Packed prefill of ``tasks`` (any mix of lengths).  Each request recomputes positions ``[start, end)`` where
        ``start`` is where its previous chunk stopped, else ``min(cached prefix, len - 1)``, unless ``start_pos`` forces
        one value for all; ``end`` is the prompt length unless ``end_positions[task_id]`` stops the chunk earlier
        (chunked prefill).  Only requests whose chunk reaches the end of the prompt are sampled and returned.
        ``wait=False``: the second element of the result is a callable that reads the sampled tokens back."""
        tasks = sorted(tasks, key=lambda t: t.task_id)
        ids = [t.task_id for t in tasks]
        lens = [len(t.prompt_ids) for t in tasks]
        if start_pos is not None:
            starts = [start_pos] * len(tasks)
        else:
            starts = [t.prefill_pos if t.prefill_pos is not None else min(self.task_cache.task_cached(t.task_id), n - 1)
                      for t, n in zip(tasks, lens)]
        ends = [min(n, (end_positions or {}).get(t.task_id, n)) for t, n in zip(tasks, lens)]
        nothing = ([], []) if wait else ([], list)
        if any(s >= e for s, e in zip(starts, ends)):
            return nothing
        for t, s in zip(tasks, starts):
            if t.prefill_start is None:
                t.prefill_start = s
        flat_ids = [tok for t, s, e in zip(tasks, starts, ends) for tok in t.prompt_ids[s:e]]
        flat_pos = [p for s, e in zip(starts, ends) for p in range(s, e)]
        pin = self.device.type == "cuda"
        input_ids = torch.tensor(flat_ids, dtype=torch.long, pin_memory=pin).to(self.device, non_blocking=True)
        position_ids = torch.tensor(flat_pos, dtype=torch.long, pin_memory=pin).to(self.device, non_blocking=True)
        last, acc, complete = [], 0, []
        for t, s, e, n in zip(tasks, starts, ends, lens):
            acc += e - s
            t.prefill_pos = e
            if e == n:
                last.append(acc - 1)
                complete.append(t)
        with torch.inference_mode(), timed(f"execute_prefill b={len(tasks)} tokens={len(flat_ids)}", logger):
            kv = self.task_cache.bind(ids, self._workspace, start_positions=starts,
                                      end_positions=ends if end_positions is not None else None)
            fused = getattr(self.model, "supports_fused_head", False)
            out = self.model(input_ids, position_ids=position_ids, kv_cache=kv, fwd="prefill",
                             **({"return_logits": False} if fused else {}))
            if not complete:
                return nothing
            rows = torch.tensor(last, dtype=torch.long, device=self.device)
            logits = self.model.lm_head(out["hidden_states"][rows]) if fused else out["logits"][rows]
            return complete, self._sample(logits, complete, return_logprobs, wait=wait)

    # -- decode -------------------------------------------------------------------------------------------------------------
    def execute_decode(self, tasks: List[Task], return_logprobs: bool = False, wait: bool = True):
        """One token for every task.  ``wait=False`` returns a callable that reads the sampled tokens back."""
        if not tasks:
            return [] if wait else list
        b, ws = len(tasks), self._workspace
        tokens = ws.fill_input_ids([t.output_ids[-1] if t.output_ids else t.prompt_ids[-1] for t in tasks])
        ids = [t.task_id for t in tasks]
        positions = [t.next_pos for t in tasks]
        kv = self.task_cache.bind(ids, ws)
        sig = tuple(ids)
        steady = self.task_cache.bind_was_steady and self._decode_cache is not None and self._decode_cache.task_sig == sig
        if steady:
            info = self._decode_cache.sampling_info
            ws.position_ids[:b] += 1
        else:
            info = build_sampling_info(tasks, self.device)
            ws.put_long(ws.position_ids, positions)
        self._decode_cache = DecodeSteadyState(sig, positions, info)
        from astrai_b200.ops import backend as attn_backends

        use_graph = self.cuda_graph_enabled and attn_backends.get_backend(self.device.type) is self._graph_backend
        with torch.inference_mode(), timed(f"execute_decode forward b={b}", logger):
            if use_graph:
                rows = self._bucket(b)
                if not steady:
                    self._zero_padding(b, rows)
                out = self._graph_ctx.forward(self.model, key=(rows,), input_ids=ws.input_ids[:rows], kv_cache=self._padded(kv, b, rows),
                                              position_ids=ws.position_ids[:rows], fwd="decode")
            else:
                out = self.model(input_ids=tokens, kv_cache=kv, position_ids=ws.position_ids[:b], fwd="decode")
            return self._sample(out["logits"][:b], tasks, return_logprobs, info=info, wait=wait)
