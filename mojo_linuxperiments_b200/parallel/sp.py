"""Token-sharded ("sequence parallel") tensor-parallel linears fused with their collectives.

Between transformer blocks rank r owns token rows [r*R, (r+1)*R) with R = ceil(M / world).  Two ops move between that
layout and the all-tokens / own-heads layout attention and the FFN inner dimension need:

  ``ag_linear``  all-gather -> GEMM (column-parallel QKV, gate|up): the GEMM kernel's comm warps push this rank's
                 int8 rows and scales into every rank's gather buffer while its tensor-core warps consume the rows
                 that have already arrived (``csrc/kernels/w8a8_gemm_tp.cu``, gather form);
  ``rs_linear``  GEMM -> reduce-scatter (row-parallel o_proj, down): the GEMM epilogue stores its bf16 tiles into the
                 owner's receive slots and the same kernel sums the world slots of its own rows (scatter form).

``SPLink`` carries one rank's view of the buffers.  ``SPLink.on_heap`` places them in a ``SymmetricHeap`` (real
multi-GPU use); ``virtual_links`` builds ``world`` links over ordinary buffers of ONE device, which lets the tests and
the single-GPU profile run every rank's kernels one after another (phase masks keep kernels from waiting on launches
that have not happened yet).  The reference has no counterpart: its only collectives are the chain / butterfly sums of
``test_linux_threading.mojo:400-553``.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import torch

from ..ops import _lib

PHASE_ALL, PHASE_TILES, PHASE_TAIL, PHASE_PUSH = 7, 1, 2, 4
EP_KMAX = 8                  # routing slots per token in the dispatch buffers


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


@dataclass
class SPLayout:
    """Byte offsets of the exchange areas inside every rank's heap (identical on all ranks)."""
    world: int
    m_cap: int
    k_cap: int
    n_cap: int
    r_cap: int = 0
    blk_cap: int = 0
    q_off: tuple = ()
    s_off: tuple = ()
    flag_off: int = 0
    done_off: int = 0
    recv_off: tuple = ()
    ctr_off: int = 0
    ids_off: tuple = ()        # expert routing lists of all tokens (int32 / fp32, 8 per token), per parity
    wts_off: tuple = ()
    nbytes: int = 0

    def __post_init__(self):
        self.r_cap = (self.m_cap + self.world - 1) // self.world
        self.blk_cap = (self.r_cap + 127) // 128
        off = 0

        def take(n, align=1024):
            nonlocal off
            start = _round_up(off, align)
            off = start + n
            return start
        self.q_off = (take(self.m_cap * self.k_cap), take(self.m_cap * self.k_cap))
        self.s_off = (take(self.m_cap * 4), take(self.m_cap * 4))
        self.flag_off = take(self.world * self.blk_cap * 4)
        self.done_off = take(self.world * 4)
        self.recv_off = (take(self.world * self.r_cap * self.n_cap * 2), take(self.world * self.r_cap * self.n_cap * 2))
        self.ctr_off = take(16)
        self.ids_off = (take(self.m_cap * EP_KMAX * 4), take(self.m_cap * EP_KMAX * 4))
        self.wts_off = (take(self.m_cap * EP_KMAX * 4), take(self.m_cap * EP_KMAX * 4))
        self.nbytes = _round_up(off, 1024)


@dataclass
class SPLink:
    layout: SPLayout
    rank: int
    data_ptrs: list            # every rank's heap base as mapped on this device
    mc_ptr: int                # NVLS multicast mapping of the heap (0: plain peer stores)
    base_off: int              # offset of the layout inside the heap
    device: torch.device
    limit_ms: int = 2000
    ag_words: torch.Tensor = field(default=None, repr=False)
    rs_words: torch.Tensor = field(default=None, repr=False)
    row_ctr: torch.Tensor = field(default=None, repr=False)
    status: torch.Tensor = field(default=None, repr=False)
    _keep: object = field(default=None, repr=False)

    def __post_init__(self):
        self.world = self.layout.world
        self._c_data = (ctypes.c_void_p * self.world)(*self.data_ptrs)
        z = lambda n: torch.zeros(n, dtype=torch.int32, device=self.device)
        self.ag_words, self.rs_words, self.row_ctr, self.status = z(4), z(4), z(max(self.layout.blk_cap, 1)), z(4)
        self.ep_blk_ctr = z(max(self.world * self.layout.blk_cap, 1))

    @classmethod
    def on_heap(cls, heap, m_cap: int, k_cap: int, n_cap: int, use_nvls: bool = True, limit_ms: int = 2000) -> "SPLink":
        lay = SPLayout(heap.world, m_cap, k_cap, n_cap)
        base = heap.alloc(lay.nbytes, align=1024)
        return cls(lay, heap.rank, list(heap.data_ptrs), heap.mc_data_ptr if (use_nvls and heap.has_multicast) else 0,
                   base, heap.device, limit_ms, _keep=heap)

    def rows_per_rank(self, M: int) -> int:
        return (M + self.world - 1) // self.world

    def my_rows(self, M: int) -> tuple[int, int]:
        """[first, last) global token rows this rank owns for an M-token call."""
        R = self.rows_per_rank(M)
        a = min(M, self.rank * R)
        return a, min(M, a + R)

    def check_status(self):
        code = int(self.status[0].item())
        if code:
            self.status.zero_()
            raise RuntimeError(f"sequence-parallel kernel status {code & 0xff} (5: a peer's flag never arrived; "
                               f"1-4: pipeline wait of GEMM family {code >> 8})")

    # ------------------------------------------------------------------------------------------------------------
    def ag_linear(self, xq_local: torch.Tensor, sx_local: torch.Tensor, wq: torch.Tensor, sw: torch.Tensor, M: int,
                  out: torch.Tensor | None = None, finish: bool = True, phase: int = PHASE_ALL) -> torch.Tensor:
        """y[M, N] = all_gather_rows(xq_local)[M, K] @ wq[N, K]^T * scales.  ``xq_local`` holds the rows this rank owns
        (``my_rows(M)``), int8 [rows, K] contiguous, ``sx_local`` their fp32 scales."""
        lay = self.layout
        K = xq_local.shape[1]
        N = wq.shape[0]
        a, b = self.my_rows(M)
        assert xq_local.dtype == torch.int8 and xq_local.is_contiguous() and xq_local.shape[0] >= b - a
        assert wq.is_contiguous() and wq.shape[1] == K and M <= lay.m_cap and K <= lay.k_cap
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=xq_local.device)
        bo = self.base_off
        rc = _lib.lib().b200_w8a8_gemm_ag(
            xq_local.data_ptr(), sx_local.data_ptr(), wq.data_ptr(), sw.data_ptr(), out.data_ptr(), M, N, K,
            out.stride(0), self.rows_per_rank(M), self._c_data, self.mc_ptr or None, self.world, self.rank,
            bo + lay.q_off[0], bo + lay.q_off[1], bo + lay.s_off[0], bo + lay.s_off[1], bo + lay.flag_off,
            bo + lay.done_off, lay.blk_cap, lay.m_cap, self.ag_words.data_ptr(), self.row_ctr.data_ptr(),
            1 if finish else 0, phase, self.status.data_ptr(), self.limit_ms, _lib.num_sms(xq_local.device.index),
            _lib.stream())
        _lib.check(rc, "w8a8_gemm_ag")
        return out

    def rs_linear(self, xq: torch.Tensor, sx: torch.Tensor, wq: torch.Tensor, sw: torch.Tensor,
                  residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
                  phase: int = PHASE_ALL) -> torch.Tensor:
        """out[my rows, N] = sum over ranks of xq[M, K_shard] @ wq[N, K_shard]^T * scales (+ residual[my rows])."""
        lay = self.layout
        M, K = xq.shape
        N = wq.shape[0]
        R = self.rows_per_rank(M)
        assert xq.dtype == torch.int8 and xq.is_contiguous() and wq.is_contiguous() and wq.shape[1] == K
        assert R <= lay.r_cap and N <= lay.n_cap
        if out is None:
            out = torch.empty((R, N), dtype=torch.bfloat16, device=xq.device)
        bo = self.base_off
        rc = _lib.lib().b200_w8a8_gemm_rs(
            xq.data_ptr(), sx.data_ptr(), wq.data_ptr(), sw.data_ptr(), out.data_ptr(), _lib.ptr(residual), M, N, K,
            out.stride(0), residual.stride(0) if residual is not None else 0, R, self._c_data, self.world, self.rank,
            bo + lay.recv_off[0], bo + lay.recv_off[1], bo + lay.ctr_off, lay.r_cap, self.rs_words.data_ptr(), phase,
            self.status.data_ptr(), self.limit_ms, _lib.num_sms(xq.device.index), _lib.stream())
        _lib.check(rc, "w8a8_gemm_rs")
        return out

    def ag_sync(self, M: int, wait: bool, finish: bool):
        lay = self.layout
        bo = self.base_off
        rc = _lib.lib().b200_ag_sync(self._c_data, self.world, self.rank, bo + lay.flag_off, bo + lay.done_off,
                                     lay.blk_cap, self.rows_per_rank(M), M, self.ag_words.data_ptr(),
                                     1 if wait else 0, 1 if finish else 0, self.status.data_ptr(), self.limit_ms,
                                     _lib.stream())
        _lib.check(rc, "ag_sync")


    # ---- expert-parallel dispatch / combine (csrc/kernels/moe_ep.cu) ---------------------------------------------
    def ep_dispatch(self, xq_local: torch.Tensor, sx_local: torch.Tensor, ids_local: torch.Tensor, wts_local: torch.Tensor,
                    M: int, experts_per_rank: int) -> None:
        """Send this rank's token rows to the ranks that own one of their top-k experts and the routing lists to all."""
        lay, bo = self.layout, self.base_off
        K, k = xq_local.shape[1], ids_local.shape[1]
        assert xq_local.is_contiguous() and ids_local.is_contiguous() and wts_local.is_contiguous()
        assert ids_local.dtype == torch.int32 and wts_local.dtype == torch.float32 and k <= EP_KMAX
        assert M <= lay.m_cap and K <= lay.k_cap
        rc = _lib.lib().b200_ep_dispatch(
            xq_local.data_ptr(), sx_local.data_ptr(), ids_local.data_ptr(), wts_local.data_ptr(), M, K, k,
            experts_per_rank, self.rows_per_rank(M), self._c_data, self.world, self.rank, bo + lay.q_off[0],
            bo + lay.q_off[1], bo + lay.s_off[0], bo + lay.s_off[1], bo + lay.ids_off[0], bo + lay.ids_off[1],
            bo + lay.wts_off[0], bo + lay.wts_off[1], bo + lay.flag_off, bo + lay.done_off, lay.blk_cap,
            self.ag_words.data_ptr(), self.row_ctr.data_ptr(), self.status.data_ptr(), self.limit_ms, _lib.stream())
        _lib.check(rc, "ep_dispatch")

    def ep_wait(self, M: int, k: int):
        """Wait for every rank's dispatch; returns the routing of all M tokens (ids int32 [M,k], weights fp32 [M,k])."""
        lay, bo = self.layout, self.base_off
        ids = torch.empty((M, k), dtype=torch.int32, device=self.device)
        wts = torch.empty((M, k), dtype=torch.float32, device=self.device)
        rc = _lib.lib().b200_ep_wait(self._c_data, self.world, self.rank, bo + lay.ids_off[0], bo + lay.ids_off[1],
                                     bo + lay.wts_off[0], bo + lay.wts_off[1], bo + lay.flag_off, lay.blk_cap,
                                     self.rows_per_rank(M), M, k, self.ag_words.data_ptr(), ids.data_ptr(),
                                     wts.data_ptr(), self.status.data_ptr(), self.limit_ms, _lib.stream())
        _lib.check(rc, "ep_wait")
        return ids, wts

    def ep_gather(self, work, d: int):
        """Rows of the dispatched tokens in this rank's slot order (the `moe_gather` of the gather buffer)."""
        lay, bo = self.layout, self.base_off
        xp = torch.empty((work.max_slots, d), dtype=torch.int8, device=self.device)
        sp_ = torch.empty((work.max_slots,), dtype=torch.float32, device=self.device)
        rc = _lib.lib().b200_ep_gather(self.data_ptrs[self.rank], bo + lay.q_off[0], bo + lay.q_off[1], bo + lay.s_off[0],
                                       bo + lay.s_off[1], self.ag_words.data_ptr(), d, work.slot_token.data_ptr(),
                                       work.meta.data_ptr(), work.max_slots, xp.data_ptr(), sp_.data_ptr(), _lib.stream())
        _lib.check(rc, "ep_gather")
        return xp, sp_

    def ep_combine(self, y: torch.Tensor, work, wts_all: torch.Tensor, ids_local: torch.Tensor, M: int,
                   experts_per_rank: int, out: torch.Tensor | None = None, phase: int = PHASE_ALL) -> torch.Tensor:
        """Weighted expert outputs back to the tokens' owners; returns out[my rows, d] (sum over contributing ranks).
        ``phase`` PHASE_TILES = scatter only, PHASE_TAIL = owner-side reduction only (single-device tests)."""
        lay, bo = self.layout, self.base_off
        d, k = y.shape[1], wts_all.shape[1]
        R = self.rows_per_rank(M)
        if out is None:
            out = torch.empty((R, d), dtype=torch.bfloat16, device=self.device)
        if phase & PHASE_TILES:
            rc = _lib.lib().b200_ep_combine_scatter(
                y.data_ptr(), y.stride(0), work.inv.data_ptr(), wts_all.data_ptr(), M, k, d, R, self._c_data, self.world,
                self.rank, bo + lay.recv_off[0], bo + lay.recv_off[1], bo + lay.ctr_off, lay.r_cap,
                self.rs_words.data_ptr(), self.ep_blk_ctr.data_ptr(), lay.blk_cap, self.status.data_ptr(), self.limit_ms,
                _lib.stream())
            _lib.check(rc, "ep_combine_scatter")
        if phase & PHASE_TAIL:
            rc = _lib.lib().b200_ep_combine_reduce(
                ids_local.data_ptr(), M, k, d, experts_per_rank, R, self._c_data, self.world, self.rank,
                bo + lay.recv_off[0], bo + lay.recv_off[1], bo + lay.ctr_off, lay.r_cap, self.rs_words.data_ptr(),
                out.data_ptr(), out.stride(0), self.status.data_ptr(), self.limit_ms, _lib.num_sms(self.device.index),
                _lib.stream())
            _lib.check(rc, "ep_combine_reduce")
        return out


def virtual_links(world: int, m_cap: int, k_cap: int, n_cap: int, device=None) -> list[SPLink]:
    """``world`` ranks emulated on one device: each "heap" is an ordinary zeroed buffer, every link sees all of them."""
    device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    lay = SPLayout(world, m_cap, k_cap, n_cap)
    heaps = [torch.zeros(lay.nbytes + 1024, dtype=torch.uint8, device=device) for _ in range(world)]
    ptrs = [_round_up(h.data_ptr(), 1024) for h in heaps]
    return [SPLink(lay, r, ptrs, 0, 0, device, _keep=heaps) for r in range(world)]
