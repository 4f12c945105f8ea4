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
    def __init__(self, device: torch.device, ws_bytes: int = 64 << 20, counters: int = 1 << 16):
        self.device = device
        self.ws = torch.zeros(ws_bytes // 4, dtype=torch.int32, device=device)
        self.counters = torch.zeros(counters, dtype=torch.int32, device=device)
        self.status = torch.zeros(4, dtype=torch.int32, device=device)

    @property
    def ws_bytes(self) -> int:
        return self.ws.numel() * 4

    def check_status(self) -> None:
        """Synchronising read of the status word; raises if any kernel recorded a bounded-wait timeout."""
        code = int(self.status[0].item())
        if code != 0:
            self.status.zero_()
            kernel = {0: "?", 1: "w8a8_gemm", 2: "w8a8_gemm_decode", 3: "attn_prefill", 4: "attn_decode_tma", 5: "attn_decode_tc",
                      6: "attn_decode_tcp", 7: "rope_kv_write", 8: "attn_decode"}.get(code >> 8, "?")
            raise RuntimeError(f"kernel status {code & 255} in {kernel}: {_STATUS_NAMES.get(code & 255, 'unknown')}")


_default: dict[int, Workspace] = {}


def default_workspace(device: torch.device) -> Workspace:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _default.get(idx)
    if w is None:
        w = Workspace(torch.device("cuda", idx))
        _default[idx] = w
    return w
