"""Expert-parallel token loop: one process per GPU, every rank decodes its own
batch of sequences through the whole model; the routed experts of each layer
are sharded over the ranks (expert e on rank e // (E / world)), everything else
is replicated.  Per layer the library runs the attention half and the mHC /
norm wrapping of the MoE sublayer (apus_cuda_model_attn_half / _ffn_input /
_ffn_output), and the MoE sublayer itself is `ExpertParallelMoe.forward`:
route -> all-to-all dispatch -> local experts -> all-to-all combine -> ordered
sum on the token's home rank, which is bit-identical to the single-GPU
sublayer.  torch.distributed (NCCL) only moves rows; the library and NCCL share
torch's current stream.
"""
import ctypes as C

import torch

from . import capi, check, lib
from .moe import ExpertParallelMoe


class _DevView:
    """Zero-copy torch view of device memory owned by the library."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 2}


def dev_tensor(ptr, shape, dtype=torch.float32, device="cuda"):
    typestr = {torch.float32: "<f4", torch.int64: "<i8", torch.int32: "<i4"}[dtype]
    return torch.as_tensor(_DevView(ptr, shape, typestr), device=device)


class EpModel:
    """desc: ApusCudaModelDesc whose experts [e_lo, e_hi) of every layer are valid."""

    def __init__(self, desc, n_layers, n_experts, topk, dim, batch, max_pos, rank=0, world=1, group=None,
                 device="cuda"):
        L = lib()
        self.L, self.batch, self.n_layers, self.dim, self.device = L, batch, n_layers, dim, device
        per = n_experts // world
        self.h = L.apus_cuda_model_create_ep(C.byref(desc), batch, max_pos, rank * per, (rank + 1) * per)
        if not self.h:
            check(1, "apus_cuda_model_create_ep")
        self.moes = [ExpertParallelMoe(n_experts, topk, dim, rank, world, group,
                                       handle=L.apus_cuda_model_moe(self.h, i), padded=True)
                     for i in range(n_layers)]
        self.ids = dev_tensor(L.apus_cuda_model_ids(self.h), (batch,), torch.int64, device)
        self.graph = None

    def close(self):
        if self.h:
            self.L.apus_cuda_model_destroy(self.h)
            self.h = None

    def capture(self):
        """Records one step (logits + feed-back) into a CUDA graph: the library's
        kernels read the position on the device and the padded exchange has fixed
        shapes, so the same graph serves every position.  Call after at least one
        plain step (workspaces are allocated by then)."""
        L, h = self.L, self.h
        if self.graph:                                   # already recorded (the prompt does it after two positions)
            return
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        check(L.apus_cuda_use_stream(side.cuda_stream, 0), "use_stream")      # synchronises outside the capture
        g = torch.cuda.CUDAGraph()
        check(L.apus_cuda_model_capturing(h, 1), "capturing")
        try:
            with torch.cuda.graph(g, stream=side):
                self._enqueue(True, True)
        finally:
            L.apus_cuda_model_capturing(h, 0)
            torch.cuda.current_stream().wait_stream(side)
            check(L.apus_cuda_use_stream(torch.cuda.current_stream().cuda_stream, 0), "use_stream")
        self.graph = g

    def step(self, want_logits=True, feed_back=True):
        """One position of every sequence.  The ids of the step are whatever
        set_ids / the previous step's feed-back left on the device."""
        if self.graph and want_logits and feed_back:
            self.graph.replay()
            check(self.L.apus_cuda_model_note_step(self.h), "note_step")
            return
        check(self.L.apus_cuda_use_stream(torch.cuda.current_stream().cuda_stream, 0), "use_stream")
        self._enqueue(want_logits, feed_back)

    def _enqueue(self, want_logits, feed_back):
        L, h = self.L, self.h
        check(L.apus_cuda_model_begin_step(h), "begin_step")
        for i in range(self.n_layers):
            check(L.apus_cuda_model_attn_half(h, i), "attn_half")
            xp = L.apus_cuda_model_ffn_input(h, i)
            if not xp:
                check(1, "ffn_input")
            x = dev_tensor(xp, (self.batch, self.dim), torch.float32, self.device)
            out = self.moes[i].forward(x, self.ids)
            check(L.apus_cuda_model_ffn_output(h, i, out.data_ptr()), "ffn_output")
        check(L.apus_cuda_model_end_step(h, int(want_logits), int(feed_back)), "end_step")

    def set_ids(self, ids):
        """ids: int64 [batch] numpy array or torch tensor (host or device)."""
        check(self.L.apus_cuda_use_stream(torch.cuda.current_stream().cuda_stream, 0), "use_stream")
        check(self.L.apus_cuda_model_set_ids(self.h, capi.ptr(ids)), "set_ids")

    def prefill(self, prompt):
        """prompt int64 numpy [batch, n]: consumed position by position; the greedy
        token after the last position is left on the device as the next ids.  The
        first two positions run as plain launches (they size every workspace), the
        rest replay the recorded step: the prompt sits on the device, a position's
        ids are copied over whatever the step before fed back, and nothing waits on
        the host.  (The recorded step computes the head at every position; only the
        last one's pick is used.)"""
        import os
        import numpy as np
        n = prompt.shape[1]
        check(self.L.apus_cuda_use_stream(torch.cuda.current_stream().cuda_stream, 0), "use_stream")
        cols = torch.from_numpy(np.ascontiguousarray(prompt.T)).to(self.device)      # [n, batch]
        record = os.environ.get("APUS_EP_GRAPH", "1") != "0"
        for t in range(n):
            self.ids.copy_(cols[t])
            if record and t >= 2 and self.graph is None:
                try:
                    self.capture()
                except Exception:                           # keep going on plain launches
                    torch.cuda.synchronize()
                    self.graph = False
            if self.graph:
                self.step(True, True)
            else:
                self.step(want_logits=(t == n - 1), feed_back=True)
        if self.graph is False:
            self.graph = None

    def read(self, logits=None, tokens=None):
        check(self.L.apus_cuda_model_read(self.h, capi.ptr(logits), capi.ptr(tokens)), "model_read")
