"""Config 3 at size: the sparse-attention decode step over long per-sequence caches
(compressed-sparse layers: stable top-512 of 32,768 and 262,144 indexer scores, raw and
BF16-rounded so that ties are everywhere; heavily compressed layers: every one of the
8,192 entries of a 1M-token context) against the reference restatement, through the
device-resident C ABI with one cache per sequence."""
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import bench                                            # the workload's case builder
from _gpu import bf16_ulps, lib
from _oracle import P, ora
from apus_b200 import synth

pytestmark = pytest.mark.gpu


def oracle_query(c, kind):
    widen = lambda u: (u.astype(np.uint32) << 16).view(np.float32)
    ring, cache = widen(c["ring"]), widen(c["cache"])
    nb = c["nb"]
    k = min(bench.ATTN_TOPK, nb) if kind == "csa" else nb
    idx = np.empty(bench.ATTN_WIN + k, np.int32)
    idx[:bench.ATTN_WIN] = np.arange(bench.ATTN_WIN)
    if kind == "csa":
        top = np.empty(k, np.int32)
        ora().ora_topk_stable(P(c["scores"]), nb, k, P(top))
        idx[bench.ATTN_WIN:] = top + bench.ATTN_WIN
    else:
        idx[bench.ATTN_WIN:] = bench.ATTN_WIN + np.arange(nb)
    o = np.empty((bench.ATTN_H, bench.ATTN_D), np.float32)
    ora().ora_sparse_attn(P(c["q"]), P(c["sink"]), bench.ATTN_H, bench.ATTN_D, P(idx), len(idx), 1, bench.ATTN_D ** -0.5,
                          P(ring), bench.ATTN_WIN, P(cache), P(o))
    return o, idx


@pytest.mark.parametrize("kind,ctx,ties", [("csa", 131072, False), ("csa", 1048576, False), ("csa", 1048576, True),
                                           ("hca", 1048576, False), ("csa", 8192, True)])
def test_long_context_decode_step(kind, ctx, ties):
    import torch
    L = lib()
    B = 2
    dev = torch.device("cuda", 0)
    case = bench.AttnDecodeCase(L, 5, kind, ctx, B, dev)
    hosts = [bench.attn_case_host(5, kind, ctx, b) for b in range(B)]
    for b in range(B):
        hosts[b]["sink"] = hosts[0]["sink"]              # the sink belongs to the layer, not the sequence
        assert np.array_equal(case.cache[b].cpu().numpy().view(np.uint16), hosts[b]["cache"])
    if ties:                                             # BF16-rounded scores: the top-512 boundary falls inside a tie group
        for b in range(B):
            hosts[b]["scores"] = synth.bf16_round(hosts[b]["scores"])
            case.scores[b].copy_(torch.from_numpy(hosts[b]["scores"]))
    case.step()
    torch.cuda.synchronize()
    assert L.apus_cuda_kernel_status(1) == 0
    got_o = case.o.cpu().numpy()
    got_idx = case.idx.cpu().numpy()
    for b in range(B):
        want_o, want_idx = oracle_query(hosts[b], kind)
        assert np.array_equal(got_idx[b], want_idx), f"sequence {b}: selected positions differ"
        u = bf16_ulps(got_o[b], want_o)
        big = np.abs(want_o) > 1e-3 * np.abs(want_o).max()
        assert u[big].max() <= 1 and (u > 0).mean() <= 1e-3, (u[big].max(), (u > 0).mean())
