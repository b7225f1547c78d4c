"""Per-tile timeline of the fused kernel (``apk_set_trace`` in include/apk.h).

The reference can only time whole ops (``torch.profiler.record_function`` around each,
autoparallel/asynctp_ops.py:741, :1077); here one kernel does the work of its pipelines, so the
stamps come from inside: for every (CTA, tile) when the first load and the first MMA were
issued, how long the MMA thread waited for operands and for a free accumulator, when the
accumulator was complete, how long the epilogue waited for the peers' partials and spent
publishing flags, and when the owner had the peers' partials summed.

    from autoparallel_b200 import timeline
    with timeline.capture(device) as tl:
        torch.ops._ap_symm_mem.fused_matmul_reduce_scatter(...)
    rec = tl.records()          # int64 array [records, 16], only the records that were written
    print(timeline.summary(rec))
"""
from __future__ import annotations

import contextlib
import ctypes as C

import torch

from . import _native as nat

FIELDS = (
    "tile", "load_t", "ready_wait", "empty_wait", "mma_t", "full_wait", "tempty_wait", "commit_t",
    "tfull_t", "partial_wait", "epi_end_t", "publish", "flags_t", "sums_t", "cta_begin_t", "cta_end_t",
)
F = {name: i for i, name in enumerate(FIELDS)}


class Timeline:
    def __init__(self, device: torch.device, records: int):
        self.buf = torch.zeros(records * len(FIELDS), dtype=torch.int64, device=device)
        self.device = device

    def records(self) -> torch.Tensor:
        """All slots [slots, 16] as int64 on the host (slots that no tile used are all zero)."""
        torch.cuda.synchronize(self.device)
        return self.buf.view(-1, len(FIELDS)).cpu()

    def clear(self) -> None:
        self.buf.zero_()


@contextlib.contextmanager
def capture(device: torch.device, records: int = 1 << 16):
    """Record the launches made inside the block (one launch at a time: a second launch overwrites the
    first one's records; call ``clear()`` between launches to tell them apart)."""
    tl = Timeline(device, records)
    with torch.cuda.device(device):
        nat.check(nat.lib().apk_set_trace(C.c_void_p(tl.buf.data_ptr()), tl.buf.numel() * 8))
        try:
            yield tl
        finally:
            torch.cuda.synchronize(device)
            nat.check(nat.lib().apk_set_trace(None, 0))


def summary(rec: torch.Tensor, sm_mhz: float = 1965.0) -> dict:
    """Kernel span and where the MMA thread's time went, from ``Timeline.records()``."""
    used = rec[rec[:, F["tile"]] > 0]
    # record 0 of every CTA carries begin / end in ns, record 1 the same instants in SM cycles
    is_first = torch.zeros(rec.shape[0], dtype=torch.bool)
    first_idx = (rec[:, F["cta_end_t"]] > 0).nonzero().flatten()
    is_first[first_idx[0::2]] = True if first_idx.numel() else False
    begin = rec[is_first, F["cta_begin_t"]]
    end = rec[is_first, F["cta_end_t"]]
    out = {"tiles": int(used.shape[0])}
    if begin.numel() and end.numel():
        out["span_us"] = (int(end.max()) - int(begin.min())) / 1e3
        nxt = first_idx[1::2]
        if nxt.numel() == begin.numel():
            cyc = (rec[nxt, F["cta_end_t"]] - rec[nxt, F["cta_begin_t"]]).double()
            ns = (end - begin).double()
            out["sm_mhz_in_kernel"] = float((cyc / ns).median()) * 1e3
            sm_mhz = out["sm_mhz_in_kernel"]
    mma = used[used[:, F["mma_t"]] > 0]
    if mma.numel():
        ctas = max(1, int(begin.numel()))
        cyc_to_us = 1.0 / sm_mhz
        out["mma_threads"] = int((mma[:, F["mma_t"]] > 0).sum())
        out["full_wait_us_per_cta"] = float(mma[:, F["full_wait"]].sum()) * cyc_to_us / ctas
        out["tempty_wait_us_per_cta"] = float(mma[:, F["tempty_wait"]].sum()) * cyc_to_us / ctas
    if used.numel():
        ctas = max(1, int(begin.numel()))
        cyc_to_us = 1.0 / sm_mhz
        out["producer_ready_wait_us_per_cta"] = float(used[:, F["ready_wait"]].sum()) * cyc_to_us / ctas
        out["producer_empty_wait_us_per_cta"] = float(used[:, F["empty_wait"]].sum()) * cyc_to_us / ctas
        out["epilogue_partial_wait_us_per_cta"] = float(used[:, F["partial_wait"]].sum()) * cyc_to_us / ctas
        out["epilogue_publish_us_per_cta"] = float(used[:, F["publish"]].sum()) * cyc_to_us / ctas
    return out
