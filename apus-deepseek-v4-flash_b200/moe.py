"""Host side of the MoE sublayer: the reference's operator interface
(`apus_moe_forward`, c/moe.h:82) on HBM-resident weights, single-GPU and
expert-parallel.

Expert parallelism (one process per GPU): expert e lives on rank
e // (E / world) — contiguous blocks, the rule of the vendored reference model
(reference-0731/inference/model.py:623-626).  Gate, bias and the shared expert
are replicated.  A step is

    route (local) -> dispatch all-to-all (token rows + expert ids to the ranks
    that own the experts) -> expert FFNs (local) -> combine all-to-all (expert
    outputs back to the token's home rank) -> y[t] = sum_j w[t,j]*eo[t,j] in
    slot order on the home rank + shared expert, BF16 round.

The combine sums on the token's home rank in top-k slot order, so the result
is bit-identical to the single-GPU run (the reference has no collective;
its summation order is c/moe.h:148-158).  torch.distributed is only the
plumbing: NCCL moves the rows, every arithmetic step is a kernel of
libapus_b200.so.
"""
import ctypes as C

import torch
import torch.distributed as dist

from . import capi, check, lib


def owner_ranks(eids, n_experts, world):
    """Rank that owns each expert id (contiguous partition)."""
    return torch.div(eids, n_experts // world, rounding_mode="floor")


def dispatch_plan(idx, n_experts, world):
    """From routing indices idx [s, topk] build the dispatch permutation.

    Returns (order, send_counts): `order` lists the flat routing positions
    (t*topk + j) grouped by destination rank, stable within a rank; send_counts
    [world] is how many go to each rank."""
    flat = idx.reshape(-1)
    dest = owner_ranks(flat, n_experts, world)
    order = torch.argsort(dest, stable=True)
    send_counts = torch.bincount(dest, minlength=world)
    return order, send_counts


def exchange_counts(send_counts, group=None):
    """All ranks learn how many rows each peer sends them."""
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    return recv_counts


class ExpertParallelMoe:
    """One MoE sublayer sharded over the ranks of a process group.

    `experts_fn(rows, eids) -> outs` computes the routed-expert FFN for each
    (row, global expert id) pair whose expert is local; by default it is the
    CUDA library's apus_cuda_moe_experts_dev.  Tests inject a CPU stand-in to
    exercise the exchange logic over gloo."""

    def __init__(self, n_experts, topk, dim, rank=0, world=1, group=None, handle=None,
                 experts_fn=None, route_fn=None, shared_fn=None, combine_fn=None, padded=False):
        assert n_experts % world == 0, "experts must divide evenly over the ranks"
        self.E, self.topk, self.dim = n_experts, topk, dim
        self.rank, self.world, self.group = rank, world, group
        self.handle = handle
        self.padded = padded
        self.e_lo = rank * (n_experts // world)
        self.e_hi = self.e_lo + n_experts // world
        self.experts_fn = experts_fn or self._experts_cuda
        self.route_fn = route_fn or self._route_cuda
        self.shared_fn = shared_fn or self._shared_cuda
        self.combine_fn = combine_fn or self._combine_cuda

    # ---- CUDA-library steps (device tensors, current stream) -----------------------
    @staticmethod
    def _stream():
        return torch.cuda.current_stream().cuda_stream

    _side = {}

    @classmethod
    def _side_stream(cls, device):
        """One side stream per device, shared by the sublayers (they run one after another)."""
        key = str(device)
        if key not in cls._side:
            cls._side[key] = torch.cuda.Stream(device=device)
        return cls._side[key]

    def _route_cuda(self, x, ids):
        s = x.shape[0]
        idx = torch.empty(s, self.topk, dtype=torch.int32, device=x.device)
        wgt = torch.empty(s, self.topk, dtype=torch.float32, device=x.device)
        check(lib().apus_cuda_moe_route_dev(self.handle, x.data_ptr(),
                                            ids.data_ptr() if ids is not None else None, s,
                                            idx.data_ptr(), wgt.data_ptr(), None, None,
                                            self._stream()), "moe_route_dev")
        return idx, wgt

    def _experts_cuda(self, rows, eids):
        n = rows.shape[0]
        out = torch.empty(max(n, 1), self.dim, dtype=torch.float32, device=rows.device)
        if n:
            rr = torch.arange(n, dtype=torch.int32, device=rows.device)
            check(lib().apus_cuda_moe_experts_dev(self.handle, rows.data_ptr(), n, rr.data_ptr(),
                                                  eids.data_ptr(), n, out.data_ptr(),
                                                  self._stream()), "moe_experts_dev")
        return out[:n]

    def _shared_cuda(self, x):
        out = torch.empty_like(x)
        check(lib().apus_cuda_moe_shared_dev(self.handle, x.data_ptr(), x.shape[0], out.data_ptr(),
                                             self._stream()), "moe_shared_dev")
        return out

    def _combine_cuda(self, eo, wgt, shared):
        s = wgt.shape[0]
        out = torch.empty(s, self.dim, dtype=torch.float32, device=eo.device)
        check(lib().apus_cuda_moe_combine_dev(self.handle, eo.data_ptr(), wgt.data_ptr(),
                                              shared.data_ptr(), s, out.data_ptr(), None,
                                              self._stream()), "moe_combine_dev")
        return out

    # ---- one sublayer step -------------------------------------------------------------
    def forward(self, x, ids=None):
        """x [s, dim] f32 (BF16-valued) on this rank's device -> out [s, dim]."""
        s = x.shape[0]
        if self.padded and (self.world > 1 or dist.is_initialized()):
            return self.forward_padded(x, ids)
        idx, wgt = self.route_fn(x, ids)
        if self.world == 1:
            rows = torch.arange(s, device=x.device).repeat_interleave(self.topk)
            eo = self.experts_fn(x[rows].contiguous(), idx.reshape(-1).contiguous())
            return self.combine_fn(eo.contiguous(), wgt, self.shared_fn(x))
        order, send_counts = dispatch_plan(idx.long(), self.E, self.world)
        recv_counts = exchange_counts(send_counts, self.group)
        # the split sizes of a variable all-to-all live on the host
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        tok = torch.div(order, self.topk, rounding_mode="floor")
        send_rows = x[tok].contiguous()
        send_eids = idx.reshape(-1)[order].contiguous()
        n_recv = sum(rc)
        recv_rows = torch.empty(n_recv, self.dim, dtype=x.dtype, device=x.device)
        recv_eids = torch.empty(n_recv, dtype=send_eids.dtype, device=x.device)
        dist.all_to_all_single(recv_rows, send_rows, rc, sc, group=self.group)
        dist.all_to_all_single(recv_eids, send_eids, rc, sc, group=self.group)
        shared = self.shared_fn(x)                       # overlaps the exchange on the GPU queue
        eo_recv = self.experts_fn(recv_rows, recv_eids).contiguous()
        eo_back = torch.empty(order.numel(), self.dim, dtype=x.dtype, device=x.device)
        dist.all_to_all_single(eo_back, eo_recv, sc, rc, group=self.group)
        eo = torch.empty_like(eo_back)
        eo[order] = eo_back                              # back to (t, j) order
        return self.combine_fn(eo, wgt, shared)


    def forward_padded(self, x, ids=None):
        """The same exchange with fixed shapes and no host synchronisation: every
        (source, destination) pair carries `s * topk` row slots (the worst case),
        unused slots hold expert id -1, which the expert kernels skip.  All ranks
        must bring the same number of tokens.  Nothing here depends on device
        values on the host, so a whole step can be captured into a CUDA graph."""
        s, W, dim = x.shape[0], self.world, self.dim
        # the shared expert needs nothing from the exchange: on the GPU it runs on a side
        # stream beside routing, the all-to-alls and the routed experts (a parallel branch
        # when the step is being captured into a graph)
        side = cur = None
        if x.is_cuda:
            cur = torch.cuda.current_stream()
            side = self._side_stream(x.device)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                shared = self.shared_fn(x)
        idx, wgt = self.route_fn(x, ids)
        R = s * self.topk
        C = R                                            # slots per destination
        fused = x.is_cuda and idx.dtype == torch.int32 and x.dtype == torch.float32
        if fused and self._compact_ok():
            # compact payload: a row travels as E4M3 codes + per-128 scales (quantised once, here),
            # an expert output as its BF16 bits -- 4,224 B out and 8,192 B back per routing slot
            # instead of 16,384 B each way
            L, st = lib(), self._stream()
            rb = int(L.apus_cuda_moe_ep_row_bytes(self.handle))
            send_q, recv_q, send_eids, recv_eids, eo_send, eo_back, eo, slot = self._compact_bufs(x.device, W * C, R, rb)
            check(L.apus_cuda_moe_ep_plan_dev(idx.data_ptr(), R, self.E, W, C, send_eids.data_ptr(), slot.data_ptr(), st),
                  "moe_ep_plan_dev")
            check(L.apus_cuda_moe_ep_pack_dev(self.handle, x.data_ptr(), s, slot.data_ptr(), R, send_q.data_ptr(), st),
                  "moe_ep_pack_dev")
            dist.all_to_all_single(recv_q, send_q, group=self.group)
            dist.all_to_all_single(recv_eids, send_eids, group=self.group)
            check(L.apus_cuda_moe_experts_q_dev(self.handle, recv_q.data_ptr(), W * C, recv_eids.data_ptr(),
                                                eo_send.data_ptr(), st), "moe_experts_q_dev")
            dist.all_to_all_single(eo_back, eo_send, group=self.group)
            check(L.apus_cuda_moe_ep_unpack_dev(eo_back.data_ptr(), dim, slot.data_ptr(), R, eo.data_ptr(), st),
                  "moe_ep_unpack_dev")
            cur.wait_stream(side)
            shared.record_stream(cur)
            return self.combine_fn(eo, wgt, shared)
        if fused:
            # three library kernels instead of a dozen tensor ops: slots + expert ids, rows in
            send_rows, send_eids, recv_rows, recv_eids, eo_back, eo, slot = self._exchange_bufs(x.device, W * C, R)
            st = self._stream()
            check(lib().apus_cuda_moe_ep_plan_dev(idx.data_ptr(), R, self.E, W, C, send_eids.data_ptr(),
                                                  slot.data_ptr(), st), "moe_ep_plan_dev")
            check(lib().apus_cuda_moe_ep_rows_dev(x.data_ptr(), dim, slot.data_ptr(), R, self.topk, 0,
                                                  send_rows.data_ptr(), st), "moe_ep_rows_dev")
        else:
            flat = idx.reshape(-1).long()
            dest = owner_ranks(flat, self.E, W)
            order = torch.argsort(dest, stable=True)
            dest_s = dest[order]
            ranks = torch.arange(W, device=x.device)
            counts = (dest_s[:, None] == ranks[None, :]).sum(0)
            starts = torch.cumsum(counts, 0) - counts
            slot = dest_s * C + (torch.arange(R, device=x.device) - starts[dest_s])
            send_rows = torch.zeros(W * C, dim, dtype=x.dtype, device=x.device)
            send_eids = torch.full((W * C,), -1, dtype=idx.dtype, device=x.device)
            send_rows[slot] = x[torch.div(order, self.topk, rounding_mode="floor")]
            send_eids[slot] = idx.reshape(-1)[order]
            recv_rows = torch.empty_like(send_rows)
            recv_eids = torch.empty_like(send_eids)
        dist.all_to_all_single(recv_rows, send_rows, group=self.group)
        dist.all_to_all_single(recv_eids, send_eids, group=self.group)
        if side is None:
            shared = self.shared_fn(x)
        eo_recv = self.experts_fn(recv_rows, recv_eids).contiguous()
        if fused:
            dist.all_to_all_single(eo_back, eo_recv, group=self.group)
            check(lib().apus_cuda_moe_ep_rows_dev(eo_back.data_ptr(), dim, slot.data_ptr(), R, self.topk, 1,
                                                  eo.data_ptr(), self._stream()), "moe_ep_rows_dev")
        else:
            eo_back = torch.empty_like(eo_recv)
            dist.all_to_all_single(eo_back, eo_recv, group=self.group)
            eo = torch.empty(R, dim, dtype=x.dtype, device=x.device)
            eo[order] = eo_back[slot]                    # back to (t, j) order
        if side is not None:
            cur.wait_stream(side)
            shared.record_stream(cur)
        return self.combine_fn(eo, wgt, shared)

    _bufs = {}

    def _compact_ok(self):
        """The compact payload needs the library's own expert path on the tcgen05 kernels."""
        ok = getattr(self, "_compact", None)
        if ok is None:
            import os
            ok = (self.handle is not None and self.experts_fn == self._experts_cuda
                  and os.environ.get("APUS_EP_COMPACT", "1") != "0"
                  and lib().apus_cuda_moe_use_tc(self.handle, -1) == 1)
            self._compact = ok
        return ok

    def _compact_bufs(self, device, n_slots, n_rout, row_bytes):
        key = ("q", str(device), n_slots, n_rout, self.dim, row_bytes)
        b = ExpertParallelMoe._bufs.get(key)
        if b is None:
            u8 = dict(dtype=torch.uint8, device=device)
            i32 = dict(dtype=torch.int32, device=device)
            i16 = dict(dtype=torch.bfloat16, device=device)      # BF16 bits (NCCL has no 16-bit integer type)
            b = (torch.zeros(n_slots, row_bytes, **u8), torch.empty(n_slots, row_bytes, **u8), torch.empty(n_slots, **i32),
                 torch.empty(n_slots, **i32), torch.zeros(n_slots, self.dim, **i16), torch.empty(n_slots, self.dim, **i16),
                 torch.empty(n_rout, self.dim, dtype=torch.float32, device=device), torch.empty(n_rout, **i32))
            ExpertParallelMoe._bufs[key] = b
        return b

    def _exchange_bufs(self, device, n_slots, n_rout):
        """Exchange buffers, kept per (device, shape) and shared by the sublayers, which run
        one after another on one stream.  Unused row slots are never read by the expert
        kernels (their expert id is -1), so the rows are not cleared between uses."""
        key = (str(device), n_slots, n_rout, self.dim)
        b = ExpertParallelMoe._bufs.get(key)
        if b is None:
            f = dict(dtype=torch.float32, device=device)
            i = dict(dtype=torch.int32, device=device)
            b = (torch.zeros(n_slots, self.dim, **f), torch.empty(n_slots, **i), torch.empty(n_slots, self.dim, **f),
                 torch.empty(n_slots, **i), torch.empty(n_slots, self.dim, **f), torch.empty(n_rout, self.dim, **f),
                 torch.empty(n_rout, **i))
            ExpertParallelMoe._bufs[key] = b
        return b


def create_handle(moew, e_lo, e_hi):
    """Upload the experts [e_lo, e_hi) of an ApusMoeW (plus gate/shared) to HBM."""
    h = lib().apus_cuda_moe_create(C.byref(moew), e_lo, e_hi)
    if not h:
        check(1, "apus_cuda_moe_create")
    return h
