"""Expert-parallel token exchange over NVLink peer memory.

Two primitives, each one peer-store pass plus one bounded barrier on the stream:

* ``dispatch``: rows sorted by global expert on every source rank -> expert-major compact rows on the rank that owns
  the experts (the A operand of the ragged grouped GEMM).
* ``return_rows``: compact rows -> back on the source rank, in the source's sorted order.

The backward of one is the other.  Receive windows hold ``cap`` rows per source (the most a source can send: all of
its tokens x top_k), so nothing is ever sized from data on the host.  The expert activations are allocated for the same
bound (``ep * cap`` rows; ``KF_EP_EXACT_ROWS=1`` restores the exact allocation at the price of one 4-byte host read per
layer): the grouped kernels and the move kernels take their row ranges from device-side offsets, so the unused tail of
those buffers is never read or written and no step of the exchange waits for the host.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from kempnerforge_b200.comm.symmetric import SymmBuffer
from kempnerforge_b200.ops import cuda as kc


class EPContext:
    def __init__(self, group, device: torch.device, cap_rows: int, cols: int, n_local: int) -> None:
        self.group = group
        self.ep = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.cap, self.cols, self.n_local = cap_rows, cols, n_local
        self.windows = SymmBuffer(self.ep * cap_rows * cols, torch.bfloat16, device, group)
        self.returns = SymmBuffer(cap_rows * cols, torch.bfloat16, device, group)
        self.table = SymmBuffer(self.ep * (n_local + 1), torch.int32, device, group)
        self.window_ptrs = (ctypes.c_longlong * 8)(*self.windows.peer_ptrs)
        self.return_ptrs = (ctypes.c_longlong * 8)(*self.returns.peer_ptrs)
        self.table_ptrs = (ctypes.c_longlong * 8)(*self.table.peer_ptrs)
        self.windows.barrier()

    def fits(self, rows: int, cols: int, n_local: int) -> bool:
        return rows <= self.cap and cols <= self.cols and n_local == self.n_local

    # ---- raw passes ------------------------------------------------------------------------------------
    def put(self, src: torch.Tensor, slot_of_row, k: int, offsets_g: torch.Tensor, max_rows: int) -> None:
        L = kc.lib()
        kc._check(L.kf_ep_put_bf16(src.data_ptr(), slot_of_row.data_ptr() if slot_of_row is not None else None, k,
                                   offsets_g.data_ptr(), self.n_local, self.ep, self.rank, src.shape[1], self.cap,
                                   self.window_ptrs, self.table_ptrs, max_rows, kc._stream()), "kf_ep_put_bf16")
        self.windows.barrier()

    def layout(self):
        dev = self.table.tensor.device
        offsets_l = torch.empty(self.n_local + 1, dtype=torch.int32, device=dev)
        chunk_dst = torch.empty(self.ep * self.n_local, dtype=torch.int32, device=dev)
        chunk_src = torch.empty_like(chunk_dst)
        total = torch.empty(1, dtype=torch.int32, device=dev)
        table = self.table.tensor.clone()  # later calls overwrite the symmetric table; the backward needs this one
        kc._check(kc.lib().kf_ep_layout(table.data_ptr(), self.ep, self.n_local, offsets_l.data_ptr(),
                                        chunk_dst.data_ptr(), chunk_src.data_ptr(), total.data_ptr(), kc._stream()),
                  "kf_ep_layout")
        exact = os.environ.get("KF_EP_EXACT_ROWS", "0") == "1"
        return {"table": table, "offsets_l": offsets_l, "chunk_dst": chunk_dst, "chunk_src": chunk_src,
                "total": int(total.item()) if exact else self.ep * self.cap}  # rows to allocate (exact or the bound)

    def compact(self, lay: dict, cols: int) -> torch.Tensor:
        out = torch.empty((lay["total"], cols), dtype=torch.bfloat16, device=self.table.tensor.device)
        kc._check(kc.lib().kf_ep_move_bf16(self.windows.tensor.data_ptr(), out.data_ptr(), lay["table"].data_ptr(),
                                           lay["chunk_dst"].data_ptr(), lay["chunk_src"].data_ptr(), self.ep, self.n_local,
                                           cols, self.cap, 1, None, kc._stream()), "kf_ep_move_bf16")
        return out

    def send_back(self, compact: torch.Tensor, lay: dict, n_sorted: int) -> torch.Tensor:
        cols = compact.shape[1]
        kc._check(kc.lib().kf_ep_move_bf16(None, compact.data_ptr(), lay["table"].data_ptr(), lay["chunk_dst"].data_ptr(),
                                           lay["chunk_src"].data_ptr(), self.ep, self.n_local, cols, self.cap, 0,
                                           self.return_ptrs, kc._stream()), "kf_ep_move_bf16")
        self.returns.barrier()
        return self.returns.tensor[: n_sorted * cols].view(n_sorted, cols).clone()


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, slot_of_row, row_of_slot, k, offsets_g, ep: EPContext, holder: dict):
        x = x.contiguous()
        n_sorted = slot_of_row.numel()
        ep.put(x, slot_of_row, k, offsets_g, n_sorted)
        lay = ep.layout()
        holder["lay"] = lay  # the caller needs the routing of this call for ``return_rows``
        out = ep.compact(lay, x.shape[1])
        ctx.ep, ctx.lay, ctx.k, ctx.tokens, ctx.n_sorted = ep, lay, k, x.shape[0], n_sorted
        ctx.save_for_backward(row_of_slot)
        ctx.mark_non_differentiable(lay["offsets_l"])
        return out, lay["offsets_l"]

    @staticmethod
    def backward(ctx, d_compact, _):
        (row_of_slot,) = ctx.saved_tensors
        d_sorted = ctx.ep.send_back(d_compact.contiguous(), ctx.lay, ctx.n_sorted)
        dx = kc.moe_combine(d_sorted, row_of_slot, None, ctx.tokens, ctx.k)  # sum over the k copies of every token
        return dx, None, None, None, None, None, None


class _ReturnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_compact, offsets_g, n_sorted, lay, ep: EPContext):
        ctx.ep, ctx.lay, ctx.n_sorted = ep, lay, n_sorted
        ctx.save_for_backward(offsets_g)
        return ep.send_back(y_compact.contiguous(), lay, n_sorted)

    @staticmethod
    def backward(ctx, d_sorted):
        (offsets_g,) = ctx.saved_tensors
        ep = ctx.ep
        ep.put(d_sorted.contiguous(), None, 1, offsets_g, ctx.n_sorted)
        # same routing as the forward: the table the peers just rewrote equals the saved one
        return ep.compact(ctx.lay, d_sorted.shape[1]), None, None, None, None


def dispatch(x, slot_of_row, row_of_slot, k, offsets_g, ep: EPContext):
    """(compact expert-major rows on the owner rank, int32 offsets of its local experts, layout for ``return_rows``)."""
    holder: dict = {}
    out, offsets_l = _DispatchFn.apply(x, slot_of_row, row_of_slot, k, offsets_g, ep, holder)
    return out, offsets_l, holder["lay"]


def return_rows(y_compact, offsets_g, n_sorted, lay, ep: EPContext):
    return _ReturnFn.apply(y_compact, offsets_g, n_sorted, lay, ep)
