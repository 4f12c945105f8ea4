"""Per-device scratch the kernels share: stream-K partial sums, tile counters, the status word.

Kernels leave the scratch zeroed when they finish, so one buffer serves every launch on a stream; launches
that may overlap on the GPU (different streams) must use different ``Workspace`` objects.
"""
from __future__ import annotations

import torch

_STATUS_NAMES = {
    0: "ok", 1: "timeout: shared-memory stage never filled", 2: "timeout: shared-memory stage never released",
    3: "timeout: accumulator never completed", 4: "timeout: accumulator never drained",
    5: "timeout: flag from a peer never arrived", 6: "bad argument", 7: "timeout while draining",
}


class Workspace:
    DEFAULT_WS_BYTES = 64 << 20
    DEFAULT_COUNTERS = 1 << 16

    @classmethod
    def nbytes(cls, ws_bytes: int | None = None, counters: int | None = None) -> int:
        return (ws_bytes or cls.DEFAULT_WS_BYTES) + 4 * (counters or cls.DEFAULT_COUNTERS) + 16 + 256 + 16 + 5 * 1024

    def __init__(self, device: torch.device, ws_bytes: int = 64 << 20, counters: int = 1 << 16, alloc=None):
        """``alloc(shape, dtype) -> zeroed tensor`` places the buffers (e.g. in a rank's HBM arena); default torch."""
        if alloc is None:
            def alloc(shape, dtype):
                return torch.zeros(shape, dtype=dtype, device=device)
        self.device = device
        self.ws = alloc((ws_bytes // 4,), torch.int32)
        self.counters = alloc((counters,), torch.int32)
        self.status = alloc((4,), torch.int32)
        # fused activation prologue of the decode GEMMs: one flag word per token row, and the step word whose change
        # between two replays of a captured launch keeps a replay from mistaking last step's flags for its own
        self.qflags = alloc((64,), torch.int32)
        self.step = alloc((4,), torch.int32)

    def next_step(self) -> None:
        """Advance the step word (a tiny device-side add on the current stream): call once per forward pass."""
        self.step.add_(1)

    @property
    def ws_bytes(self) -> int:
        return self.ws.numel() * 4

    def check_status(self) -> None:
        """Synchronising read of the status word; raises if any kernel recorded a bounded-wait timeout."""
        st = self.status.tolist()
        code = st[0]
        if st[1] != 0:
            self.status.zero_()
            raise RuntimeError(f"range-checked kernel refused heap offset {(st[3] & 0xffffffff) << 32 | (st[2] & 0xffffffff)}: "
                               "the access was skipped")
        if code != 0:
            self.status.zero_()
            kernel = {0: "?", 1: "w8a8_gemm", 2: "w8a8_gemm_decode", 3: "attn_prefill", 4: "attn_decode_tma", 5: "attn_decode_tc",
                      6: "attn_decode_tcp", 7: "rope_kv_write", 8: "attn_decode"}.get(code >> 8, "?")
            raise RuntimeError(f"kernel status {code & 255} in {kernel}: {_STATUS_NAMES.get(code & 255, 'unknown')}")


_default: dict[int, Workspace] = {}


def install_default_workspace(device: torch.device, w: Workspace) -> None:
    """Make ``w`` the workspace every op on ``device`` uses from now on (the engine installs an arena-backed one)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    _default[idx] = w


def has_default_workspace(device: torch.device) -> bool:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    return idx in _default


def default_workspace(device: torch.device) -> Workspace:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _default.get(idx)
    if w is None:
        w = Workspace(torch.device("cuda", idx))
        _default[idx] = w
    return w
