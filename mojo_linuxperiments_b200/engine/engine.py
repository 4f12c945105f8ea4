"""Per-rank inference engine: admission into the paged KV cache, prefill, CUDA-graph decode steps, greedy sampling.

The decode step of a batch is captured once per batch size as one CUDA graph; replaying it is the analogue of the
reference's ``ThreadPool.launch`` on every rank and ``wait_all`` is the event the caller synchronises on
(threading/linux_threading.mojo:103-129).  The host only reads the sampled ids.  Prefill is captured too, once per
(first sequence slot, sequences, prompt length): a prompt's ~400 kernel launches otherwise cost more host time than
the GPU needs to run them once the model is sharded over several GPUs.
"""
from __future__ import annotations

import os

import torch

from ..models.config import ModelConfig, RuntimeConfig
from ..models.decoder import Decoder, KVState
from ..models import weights as Wt
from ..ops.workspace import Workspace, default_workspace, has_default_workspace, install_default_workspace
from ..parallel.comm import Comm
from ..utils.trace import op_range
from .runtime import RankRuntime


class Engine:
    _instances = 0

    def __init__(self, cfg: ModelConfig, rt: RuntimeConfig | None = None, weights: dict | None = None, seed: int = 0,
                 device=None, comm: Comm | None = None):
        self.cfg = cfg
        self.rt = rt or RuntimeConfig()
        self.comm = comm or Comm.single()
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        # where this rank runs (host thread pinned beside its GPU) and where its long-lived buffers live (HBM arena)
        if self.rt.debug:
            from ..ops import _lib
            if not _lib.lib().b200_debug_compiled():
                raise RuntimeError("RuntimeConfig.debug needs the range-checked kernel library: set B200RT_DEBUG=1 (or "
                                   "B200RT_KERNELS=debug) before the first kernel is used")
        self.runtime = RankRuntime(self.device)
        self.heartbeat = None
        if weights is None:
            weights = Wt.random_shard(cfg, self.rt.tp, self.comm.rank, self.device, seed)
        self.tp_ctx = None
        if self.comm.world > 1 and self.rt.fused_collectives:
            from ..parallel.tp import TPContext
            self.tp_ctx = TPContext(cfg.d_model, max_tokens=self.rt.max_prefill_tokens, group=self.comm.group,
                                    device=self.device, wait_limit_ms=self.rt.wait_limit_ms)
        self.model = Decoder(cfg, self.rt, weights, self.comm, self.device, tp_ctx=self.tp_ctx)
        self.kv: KVState | None = None
        self.batch = 0
        self._graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self._prefill_graphs: dict[tuple, tuple] = {}
        self._prefill_pool = None
        self.tokens = None
        self.positions = None
        self.kernels_per_step = 0
        self._stream = torch.cuda.Stream(device=self.device)
        if self.comm.world > 1 and os.environ.get("B200RT_HEARTBEAT", "1") not in ("0", "false"):
            self._start_heartbeat()
        self._admitted = 0          # tokens per sequence the KV pages of the running batch can hold
        self._host_len = 0          # tokens per sequence already in the cache (host-side mirror of ``positions``)

    # ------------------------------------------------------------------------------------------------------
    def start_batch(self, batch: int, max_total_len: int) -> None:
        """Open a batch of ``batch`` sequence slots whose sequences may grow to ``max_total_len`` tokens.  No KV page is
        reserved here: ``prefill`` / ``admit_sequence`` take the pages a prompt needs, every decode step takes one more
        page for the sequences that cross a page boundary, ``release_sequence`` gives them back."""
        if max_total_len > self.rt.max_seq_len:
            raise ValueError(f"{max_total_len} tokens exceed max_seq_len {self.rt.max_seq_len}")
        if self.kv is None or self.kv.seq_lens.numel() != batch or self.kv.max_pages * self.rt.page_size < max_total_len:
            self.kv = None                  # free the old cache before the new one is allocated
            self._graphs.clear()
            self._prefill_graphs.clear()
            self._place_buffers(batch)
            self.kv = KVState(self.cfg, self.rt, self.device, batch, self.rt.max_seq_len, alloc=self.runtime.zeros)
            self.tokens = torch.zeros(batch, dtype=torch.int64, device=self.device)
            self.positions = torch.zeros(batch, dtype=torch.int32, device=self.device)
            self.active = torch.zeros(batch, dtype=torch.int32, device=self.device)
        else:
            # same cache, same static tensors: the captured graphs stay valid
            for s in list(self.kv.owned):
                self.kv.release(s)
            self.tokens.zero_()
            self.positions.zero_()
            self.active.zero_()
            self.kv.seq_lens.zero_()
        self.kv.flush()
        self.batch = batch
        self._admitted = max_total_len
        self._lens = [0] * batch            # tokens per slot already in the cache (host mirror of ``positions``); 0: empty
        self._host_len = 0                  # longest of them

    def _place_buffers(self, batch: int) -> None:
        """One arena per rank (the reference: one arena per node, test_linux_threading.mojo:237-250) for the KV cache of
        the new batch; the kernels' scratch / counters / status words get a small arena of their own the first time, which
        lives as long as the rank (the KV arena is replaced whenever the batch geometry changes)."""
        if not has_default_workspace(self.device) and self.runtime.make_scratch_arena(Workspace.nbytes() + (2 << 20)):
            install_default_workspace(self.device, Workspace(self.device, alloc=self.runtime.scratch_zeros))
        self.runtime.make_arena(KVState.nbytes(self.cfg, self.rt, batch, self.rt.max_seq_len) + (2 << 20))

    def _start_heartbeat(self) -> None:
        """Host-side failure detection between steps: every rank beats into the rendezvous store from a background
        thread that also watches the peers; ``decode_step`` / ``prefill`` look at its verdict before they launch, so
        a rank that has gone away turns into ``RankFailure`` on the host instead of a device-side wait that runs out."""
        try:
            import torch.distributed as dist
            from ..utils.health import Heartbeat
            store = dist.distributed_c10d._get_default_store()
            Engine._instances += 1          # every rank builds its engines in the same order: the same key prefix
            self.heartbeat = Heartbeat(store, self.comm.rank, self.comm.world, interval_s=0.2, timeout_s=5.0,
                                       prefix=f"b200rt_hb_{Engine._instances}").start(monitor=True)
        except Exception as e:
            self.runtime.notes.append(f"heartbeat not started: {type(e).__name__}: {e}")
            self.heartbeat = None

    def memory_report(self) -> dict:
        """Placement of the rank (GPU, NUMA node, pinned CPUs) and the arena's counters (used / remaining / high water)."""
        r = self.runtime.report()
        if self.kv is not None:
            r["kv_pages"] = {"total": self.kv.num_pages - 1, "in_use": self.kv.pages_in_use(), "high_water": self.kv.pages_high_water,
                             "page_tokens": self.kv.page_size}
        return r

    def prefill(self, prompts, use_graph: bool = True) -> torch.Tensor:
        """Prompts of the whole batch -> first generated token per sequence (device tensor); the engine is then ready
        for ``decode_step``.  ``prompts`` is int64 [B, S] (host or device), or a list of B one-dimensional id tensors of
        any lengths (a ragged batch: the kernels take cumulative sequence lengths).  Long batches are processed in
        groups of whole sequences so that one call never carries more than ``rt.max_prefill_tokens`` tokens; for
        equal lengths each group's forward pass is one CUDA graph (captured at first use)."""
        if self.heartbeat is not None:
            self.heartbeat.check_fast()
        if isinstance(prompts, (list, tuple)):
            lens = [int(p.numel()) for p in prompts]
            if len(set(lens)) == 1:
                prompts = torch.stack([p.reshape(-1) for p in prompts])
            else:
                return self._prefill_ragged(prompts, lens)
        B, S = prompts.shape
        if S + 1 > self._admitted:
            raise ValueError(f"a prompt of {S} tokens leaves no room to decode within the {self._admitted} admitted")
        for b in range(B):
            self.kv.admit(b, S + 1)
        self.kv.flush()
        self._prefill_equal(prompts.to(self.device, non_blocking=True), 0, use_graph)
        self.positions[:B].fill_(S)
        self.kv.seq_lens[:B].fill_(S + 1)      # the next decode step attends to the prompt plus its own token
        self.active[:B].fill_(1)
        for b in range(B):
            self._lens[b] = S
        self._host_len = max(self._lens)
        return self.tokens.clone()

    def _prefill_equal(self, ids_all: torch.Tensor, slot0: int, use_graph: bool) -> None:
        """ids_all [n, S] on the device: prefill slots slot0 .. slot0 + n - 1 (pages already admitted)."""
        n, S = ids_all.shape
        group = max(1, min(n, self.rt.max_prefill_tokens // S))
        for g0 in range(0, n, group):
            g1 = min(n, g0 + group)
            b0, b1 = slot0 + g0, slot0 + g1
            ids = ids_all[g0:g1].reshape(-1)
            if not use_graph:
                self._prefill_body(ids, b0, b1, S, self._prefill_consts(b0, b1, S))
                continue
            key = (b0, b1 - b0, S)
            entry = self._prefill_graphs.get(key)
            if entry is None:
                consts = self._prefill_consts(b0, b1, S)
                ids_buf = ids.clone()
                # once eagerly on the side stream (lazy set-up, allocator warm-up, status check), then capture
                self._stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self._stream):
                    self._prefill_body(ids_buf, b0, b1, S, consts)
                torch.cuda.current_stream().wait_stream(self._stream)
                torch.cuda.synchronize()
                self.check_status()
                if self._prefill_pool is None:
                    self._prefill_pool = torch.cuda.graph_pool_handle()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self._stream, pool=self._prefill_pool):
                    self._prefill_body(ids_buf, b0, b1, S, consts)
                entry = (g, ids_buf, consts)
                self._prefill_graphs[key] = entry
            entry[1].copy_(ids, non_blocking=True)
            entry[0].replay()

    def _prefill_ragged(self, prompts, lens) -> torch.Tensor:
        """Prompts of different lengths in one call per group: ids are concatenated, every token carries its position
        and its sequence slot, attention works on the cumulative lengths (eager launches: the shapes differ per call)."""
        B = len(prompts)
        if max(lens) + 1 > self._admitted or min(lens) < 1:
            raise ValueError(f"prompt lengths {min(lens)}..{max(lens)} do not fit the {self._admitted} admitted tokens")
        for b in range(B):
            self.kv.admit(b, lens[b] + 1)
        self.kv.flush()
        dev = self.device
        b0 = 0
        while b0 < B:
            b1, tokens = b0, 0
            while b1 < B and (b1 == b0 or tokens + lens[b1] <= self.rt.max_prefill_tokens):
                tokens += lens[b1]
                b1 += 1
            ids = torch.cat([prompts[b].reshape(-1).to(torch.int64) for b in range(b0, b1)]).to(dev, non_blocking=True)
            pos = torch.cat([torch.arange(lens[b], dtype=torch.int32) for b in range(b0, b1)]).to(dev, non_blocking=True)
            sid = torch.cat([torch.full((lens[b],), b, dtype=torch.int32) for b in range(b0, b1)]).to(dev, non_blocking=True)
            cu_host = [0]
            for b in range(b0, b1):
                cu_host.append(cu_host[-1] + lens[b])
            cu = torch.tensor(cu_host, dtype=torch.int32).to(dev, non_blocking=True)
            last = torch.tensor([c - 1 for c in cu_host[1:]], dtype=torch.int64).to(dev, non_blocking=True)
            nxt = self.model.forward(ids, pos, self.kv, mode="prefill", cu_seqlens=cu, max_len=max(lens[b0:b1]), seq_ids=sid,
                                     last_idx=last)
            self.tokens[b0:b1].copy_(nxt)
            default_workspace(self.device).next_step()
            b0 = b1
        lt = torch.tensor(lens, dtype=torch.int32).to(dev, non_blocking=True)
        self.positions[:B].copy_(lt)
        self.kv.seq_lens[:B].copy_(lt + 1)
        self.active[:B].fill_(1)
        for b in range(B):
            self._lens[b] = lens[b]
        self._host_len = max(self._lens)
        return self.tokens.clone()

    def admit_sequence(self, slot: int, prompt: torch.Tensor, use_graph: bool = True) -> torch.Tensor:
        """Between two decode steps: put a new sequence into slot ``slot`` (empty, or whose sequence is finished) of the
        running batch.  Its prompt is prefilled into freshly admitted pages, the slot's token / position / length are
        set, and the captured decode graph keeps being replayed as it is (it reads those tensors, not their values
        at capture time).  Returns the sequence's first generated token (one-element device tensor)."""
        if not 0 <= slot < self.batch:
            raise IndexError(slot)
        S = int(prompt.numel())
        if S < 1 or S + 1 > self._admitted:
            raise ValueError(f"a prompt of {S} tokens does not fit the {self._admitted} admitted tokens")
        self.kv.release(slot)
        self.kv.admit(slot, S + 1)
        self.kv.flush()
        self._prefill_equal(prompt.reshape(1, S).to(torch.int64).to(self.device, non_blocking=True), slot, use_graph)
        self.positions[slot:slot + 1].fill_(S)
        self.kv.seq_lens[slot:slot + 1].fill_(S + 1)
        self.active[slot:slot + 1].fill_(1)
        self._lens[slot] = S
        self._host_len = max(self._lens)
        return self.tokens[slot:slot + 1].clone()

    def release_sequence(self, slot: int) -> None:
        """The sequence in ``slot`` is finished: its pages go back to the free list, and the slot stays in the batch as
        an empty one (length 0, page-table row on the scratch page) until ``admit_sequence`` fills it again."""
        self.kv.release(slot)
        self.kv.flush()
        self.positions[slot:slot + 1].zero_()
        self.kv.seq_lens[slot:slot + 1].zero_()
        self.active[slot:slot + 1].zero_()
        self.tokens[slot:slot + 1].zero_()
        self._lens[slot] = 0
        self._host_len = max(self._lens)

    def _prefill_consts(self, b0: int, b1: int, S: int):
        n = b1 - b0
        dev = self.device
        return (torch.arange(S, dtype=torch.int32, device=dev).repeat(n),
                torch.arange(b0, b1, dtype=torch.int32, device=dev).repeat_interleave(S),
                torch.arange(0, (n + 1) * S, S, dtype=torch.int32, device=dev),
                torch.arange(S - 1, n * S, S, dtype=torch.int64, device=dev))

    def _prefill_body(self, ids, b0, b1, S, consts) -> None:
        positions, seq_ids, cu, last = consts
        nxt = self.model.forward(ids, positions, self.kv, mode="prefill", cu_seqlens=cu, max_len=S, seq_ids=seq_ids,
                                 last_idx=last)
        self.tokens[b0:b1].copy_(nxt)
        default_workspace(self.device).next_step()

    def _decode_body(self) -> None:
        nxt = self.model.forward(self.tokens, self.positions, self.kv, mode="decode", max_len=self.rt.max_seq_len)
        self.tokens.copy_(nxt)
        self.positions.add_(self.active)        # empty slots stay at position 0, length 0
        self.kv.seq_lens.add_(self.active)
        default_workspace(self.device).next_step()      # a launch replayed next step must not match this step's row flags

    def decode_step(self, use_graph: bool = True) -> torch.Tensor:
        """One greedy token for every sequence of the batch; returns the device tensor of new ids [B].

        Raises before anything is launched when the step would write past the KV pages admitted in ``start_batch``:
        the kernels would refuse the write as well (status word), but the host knows first."""
        if self.heartbeat is not None:
            self.heartbeat.check_fast()
        if self._host_len + 1 > self._admitted:
            raise RuntimeError(f"decode step at position {self._host_len} exceeds the {self._admitted} tokens per "
                               f"sequence admitted by start_batch")
        # this step writes token number len + 1 of every running sequence: take the page it lands on if the sequence
        # does not own it yet (once per page_size steps and sequence), and push the page table if a row changed
        for b, n in enumerate(self._lens):
            if n > 0:
                self.kv.admit(b, n + 1)
                self._lens[b] = n + 1
        self.kv.flush()
        self._host_len += 1
        if not use_graph:
            self._decode_body()
            return self.tokens
        g = self._graphs.get(self.batch)
        if g is None:
            # warm up outside capture (lazy kernel attribute set-up, allocator), restoring the state afterwards
            saved = (self.tokens.clone(), self.positions.clone(), self.kv.seq_lens.clone())
            self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream):
                self._decode_body()
            torch.cuda.current_stream().wait_stream(self._stream)
            torch.cuda.synchronize()
            self.check_status()         # a bounded wait that ran out surfaces here, before anything is captured or timed
            self.tokens.copy_(saved[0]); self.positions.copy_(saved[1]); self.kv.seq_lens.copy_(saved[2])
            g = torch.cuda.CUDAGraph()
            from ..ops import _lib
            n0 = _lib.LAUNCHES[0]
            with torch.cuda.graph(g, stream=self._stream):
                self._decode_body()
            self.kernels_per_step = _lib.LAUNCHES[0] - n0      # this library's kernels inside one replay
            self.tokens.copy_(saved[0]); self.positions.copy_(saved[1]); self.kv.seq_lens.copy_(saved[2])
            self._graphs[self.batch] = g
        with op_range(f"decode_step.bs{self.batch}"):
            g.replay()
        return self.tokens

    def close(self) -> None:
        """Release what has to go before the process group does: the captured graphs (they hold symmetric-memory
        tensors and NCCL work of the communicator), the heartbeat thread, the symmetric heap, the KV cache.  After
        ``close()`` the rank can call ``torch.distributed.destroy_process_group()`` without a graph still pinning
        the communicator's resources."""
        if self.heartbeat is not None:
            self.heartbeat.stop()
            self.heartbeat = None
        torch.cuda.synchronize(self.device)
        self._graphs.clear()
        self._prefill_graphs.clear()
        self._prefill_pool = None
        self.model._decode_scratch.clear()
        if self.tp_ctx is not None:
            self.tp_ctx.sp = None
            self.tp_ctx.heap = None
            self.tp_ctx = None
            self.model.tp_ctx = None
            if self.model.moe is not None:
                self.model.moe.tp_ctx = None
        self.kv = None
        torch.cuda.synchronize(self.device)

    def check_status(self) -> None:
        """Synchronising read of the kernels' status words; raises if a device-side wait timed out."""
        default_workspace(self.device).check_status()
        if self.tp_ctx is not None:
            self.tp_ctx.heap.check_status()
            if self.tp_ctx.sp is not None:
                self.tp_ctx.sp.check_status()

    def step_from_host(self, ids_in: torch.Tensor, ids_out: torch.Tensor) -> torch.Tensor:
        """Serving-loop form of a decode step: token ids arrive in pinned host memory (the previous step's sample,
        possibly edited by the caller), the new ids are written to pinned host memory; returns after they landed."""
        self.tokens.copy_(ids_in, non_blocking=True)
        nxt = self.decode_step()
        ids_out.copy_(nxt, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return ids_out

    def generate(self, prompts: torch.Tensor, max_new_tokens: int, use_graph: bool = True) -> torch.Tensor:
        """Greedy generation. prompts int64 [B, S] -> int64 [B, max_new_tokens] on the host."""
        B, S = prompts.shape
        self.start_batch(B, S + max_new_tokens)
        out = torch.empty((max_new_tokens, B), dtype=torch.int64, pin_memory=torch.cuda.is_available())
        first = self.prefill(prompts, use_graph)
        out[0].copy_(first, non_blocking=True)
        for t in range(1, max_new_tokens):
            nxt = self.decode_step(use_graph)
            out[t].copy_(nxt, non_blocking=True)
        torch.cuda.synchronize()
        self.check_status()
        return out.t().contiguous()
