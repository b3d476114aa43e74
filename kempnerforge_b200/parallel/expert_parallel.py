"""Expert parallelism: routed experts are partitioned over an EP group; tokens travel to the rank that
owns their expert and the results travel back.

Two layouts are supported:
  * the reference's: ``ep`` is a mesh dimension of its own, EP peers see the *same* batch and replicate
    everything except the experts;
  * ``ep_in_dp``: the EP group is (a slice of) the data-parallel group, every rank routes its *own* tokens.
Both use the same dispatch: expert ``e`` lives on rank ``e // (E / ep)``.

Dispatch steps (all index math on the device):
  1. stable sort of the (token, slot) pairs by destination rank, gather rows
  2. exchange per-(rank, local expert) counts
  3. all-to-all of the rows, receive side regrouped by local expert
  4. grouped expert FFN over the received rows
  5. all-to-all back, un-permute, weight and reduce over the k slots (fixed order, no atomics)
The ``collective`` transport uses ``all_to_all_single`` (NCCL / gloo) and needs the split sizes on the
host, i.e. one device->host read per layer; the ``symmetric`` transport (kempnerforge_b200.comm) writes rows
straight into the owner's receive buffer over NVLink with device-side offsets and no host read.

Expert parameters keep *global* names (``experts.{global_index}`` / dim-0 shards of the packed tensors,
tagged ``_kf_shard = ("ep", 0)``) so that checkpoints written under EP can be re-loaded under any EP degree.

Parity: kempnerforge/distributed/expert_parallel.py:29-379.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist
from torch import nn

from kempnerforge_b200.parallel.setup import mesh_dim


def ep_group_for(mesh, ep_in_dp: bool = False, ep_size: int | None = None):
    """(process group, size) used for expert parallelism on this mesh."""
    if mesh is None:
        return None, 1
    names = mesh.mesh_dim_names or ()
    if "ep" in names:
        g, size, _ = mesh_dim(mesh, "ep")
        return g, size
    if ep_in_dp and "dp_shard" in names:
        g, size, _ = mesh_dim(mesh, "dp_shard")
        if ep_size in (None, size):
            return g, size
    return None, 1


class _AllToAll(torch.autograd.Function):
    """Row exchange with explicit split sizes; backward runs the reverse exchange."""

    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty((sum(out_splits), *x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        back = g.new_empty((sum(ctx.in_splits), *g.shape[1:]))
        dist.all_to_all_single(back, g.contiguous(), output_split_sizes=ctx.in_splits, input_split_sizes=ctx.out_splits, group=ctx.group)
        return back, None, None, None


def all_to_all_rows(x: torch.Tensor, out_splits: list[int], in_splits: list[int], group) -> torch.Tensor:
    return _AllToAll.apply(x, out_splits, in_splits, group)


def ep_dispatch_and_compute(x_flat: torch.Tensor, weights: torch.Tensor, indices: torch.Tensor, moe) -> torch.Tensor:
    """MoE forward for one rank of an EP group.  x_flat (T, D); weights / indices (T, k)."""
    group, ep = moe.ep_group, moe.ep_world_size
    n_local = moe.num_local_experts
    t, k = indices.shape
    fused = _fused_context(moe, x_flat, t * k)
    if fused is not None:
        return _ep_forward_peer_memory(x_flat, weights, indices, moe, fused)
    flat_e = indices.reshape(-1)
    # (1) sort pairs by global expert id: destination ranks are contiguous blocks of that order
    order = torch.argsort(flat_e, stable=True)
    rows = x_flat.index_select(0, order // k)
    # (2) counts per (destination rank, local expert) -> exchange
    send_counts = torch.bincount(flat_e, minlength=ep * n_local).view(ep, n_local)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    host = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).tolist()  # the one host read of this layer
    in_splits, out_splits = [int(v) for v in host[0]], [int(v) for v in host[1]]
    # (3) rows to their owners; they arrive grouped by source rank, each group sorted by local expert
    recv = all_to_all_rows(rows, out_splits, in_splits, group)
    n_recv = recv.shape[0]
    src_of_chunk = torch.arange(ep, device=recv.device).repeat_interleave(n_local)
    exp_of_chunk = torch.arange(n_local, device=recv.device).repeat(ep)
    chunk_len = recv_counts.reshape(-1)
    local_e = torch.repeat_interleave(exp_of_chunk, chunk_len, output_size=n_recv)
    by_expert = torch.argsort(local_e, stable=True)
    counts_local = recv_counts.sum(0)
    # (4) experts
    y = moe.run_experts(recv.index_select(0, by_expert), counts_local)
    if moe.gradient_scale and moe.training:
        avg = counts_local.sum().to(y.dtype) / max(1, n_local)
        scale = avg / counts_local.clamp(min=1).to(y.dtype)
        y = y * scale[local_e[by_expert]].unsqueeze(-1)
    inv = torch.empty_like(by_expert)
    inv[by_expert] = torch.arange(n_recv, device=recv.device)
    y = y.index_select(0, inv)
    # (5) back to the senders, undo the sort, weight and reduce over the k slots
    back = all_to_all_rows(y, in_splits, out_splits, group)
    inv_order = torch.empty_like(order)
    inv_order[order] = torch.arange(order.numel(), device=order.device)
    back = back.index_select(0, inv_order).view(t, k, -1)
    del src_of_chunk
    return (back * weights.unsqueeze(-1).to(back.dtype)).sum(dim=1)


def _fused_context(moe, x_flat: torch.Tensor, n_sorted: int):
    """The peer-memory exchange context of this layer's EP group, or None when the library path must be used
    (CPU, several nodes, dtypes / options the kernels do not cover, ``KF_EP_FUSED=0``)."""
    if not (x_flat.is_cuda and x_flat.dtype == torch.bfloat16 and x_flat.shape[1] % 8 == 0):
        return None
    if os.environ.get("KF_EP_FUSED", "1") == "0" or (moe.gradient_scale and moe.training):
        return None
    if "nccl" not in str(dist.get_backend(moe.ep_group)):
        return None
    if int(os.environ.get("LOCAL_WORLD_SIZE", "0") or 0) != int(os.environ.get("WORLD_SIZE", "1")):
        return None
    from kempnerforge_b200.ops import moe_ops

    if not moe_ops.native_ok(x_flat, moe.ep_world_size * moe.num_local_experts, 1) or moe.ep_world_size > 8:
        return None
    from kempnerforge_b200.comm.fused_ep import EPContext

    key = id(moe.ep_group)
    ctx = _EP_CONTEXTS.get(key)
    if ctx is None or not ctx.fits(n_sorted, x_flat.shape[1], moe.num_local_experts):
        cap = max(n_sorted, ctx.cap if ctx is not None else 0)
        cols = max(x_flat.shape[1], ctx.cols if ctx is not None else 0)
        ctx = _EP_CONTEXTS[key] = EPContext(moe.ep_group, x_flat.device, cap, cols, moe.num_local_experts)
    return ctx if ctx.cols == x_flat.shape[1] else None


_EP_CONTEXTS: dict[int, object] = {}


def _ep_forward_peer_memory(x_flat, weights, indices, moe, ctx) -> torch.Tensor:
    """Expert-parallel forward with our kernels end to end: device-side sort by global expert, rows stored straight
    into the owners' receive windows over NVLink, ragged grouped GEMMs, rows stored back, weighted combine."""
    from kempnerforge_b200.comm import fused_ep
    from kempnerforge_b200.ops import moe_ops

    t, k = indices.shape
    e_global = moe.ep_world_size * moe.num_local_experts
    offsets_g, row_of_slot, slot_of_row = moe_ops.sort_by_expert(indices, e_global)
    x_c, offsets_l, lay = fused_ep.dispatch(x_flat, slot_of_row, row_of_slot, k, offsets_g, ctx)
    counts_l = (offsets_l[1:] - offsets_l[:-1]).to(torch.int64)
    y_c = moe.run_experts(x_c, counts_l, offsets=offsets_l)
    y_sorted = fused_ep.return_rows(y_c, offsets_g, t * k, lay, ctx)
    return moe_ops.combine_rows(y_sorted, weights, row_of_slot, slot_of_row)


def apply_expert_parallel(model: nn.Module, ep_group=None, ep_in_dp: bool = False, *, device_mesh=None) -> int:
    """Keep only this rank's experts in every MoE layer and record the EP context on the layer.

    ``ep_group`` is the expert-parallel process group; a device mesh (positionally or as ``device_mesh=``) is resolved
    to its ``ep`` dimension (``dp_shard`` with ``ep_in_dp``), and a mesh without one leaves the model unchanged.
    """
    from torch.distributed.device_mesh import DeviceMesh

    from kempnerforge_b200.models.moe import MoEMLP

    if device_mesh is not None or isinstance(ep_group, DeviceMesh):
        ep_group, size = ep_group_for(device_mesh if device_mesh is not None else ep_group, ep_in_dp)
        if size <= 1:
            return 0
    elif ep_group is None:
        return 0

    ep = dist.get_world_size(ep_group)
    rank = dist.get_rank(ep_group)
    n_layers = 0
    for module in model.modules():
        if not isinstance(module, MoEMLP):
            continue
        e = module.num_experts
        if e % ep:
            raise ValueError(f"num_experts ({e}) is not divisible by ep ({ep})")
        n_local = e // ep
        lo = rank * n_local
        if module.packed_experts:
            for name in ("up_w", "down_w", "gate_w"):
                if hasattr(module, name):
                    full = getattr(module, name)
                    local = nn.Parameter(full.detach()[lo : lo + n_local].clone(), requires_grad=full.requires_grad)
                    local._kf_shard = ("ep", 0)
                    local._kf_global_shape = tuple(full.shape)
                    setattr(module, name, local)
        else:
            kept = nn.ModuleDict({str(lo + j): module.experts[lo + j] for j in range(n_local)})
            for sub in kept.values():
                for p in sub.parameters():
                    p._kf_ep_local = True
            module.experts = kept
        module.ep_world_size = ep
        module.ep_group = ep_group
        module.local_expert_start = lo
        module.num_local_experts = n_local
        module.ep_in_dp = ep_in_dp
        n_layers += 1
    model.ep_group = ep_group
    model.ep_in_dp = ep_in_dp
    return n_layers
