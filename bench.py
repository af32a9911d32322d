#!/usr/bin/env python3
"""Benchmark of the hot path: the full DeepSeek-V4-Flash token loop (43 layers,
256 MXFP4 routed experts + FP8 shared expert per layer, vocabulary 129,280) with
random-init weights generated in HBM by the library's counter-based generator,
a 512-token prompt per sequence, then greedy decode at batch 32 (and batch 1).

    python bench.py --gpus N --steps K --warmup W            # this repository
    python bench.py --impl reference --gpus N --steps K ...  # reference C code on the host cores

One JSON line on stdout (rank 0).  `value` is whole-job decode tokens/s with the
sampled token fed back on the device; `e2e` is the same metric with HOST token ids
in and HOST sampled ids out every step (copies inside the timed region);
`roofline` describes the dominant kernel (MXFP4 gate/up expert GEMV with fused
SwiGLU) from CUDA events recorded around its launches; `cpu_baseline` is the
unmodified reference timed on the host cores in the same run; `tokens_fnv1a` is a
digest of the tokens rank 0's sequences produced -- the same prompts at every N,
so equal digests across N mean the expert-parallel loop decodes what one GPU does.

N > 1: the routed experts are sharded over the ranks (contiguous blocks), every
rank decodes its own `--batch` sequences (weak scaling; `strong_bs32` / `strong_bs1`
add the fixed-total-batch figures), dispatch and combine are NCCL all-to-alls.

Other workloads: --workload moe_layer (one MoE sublayer), fp8_gemm (config 1).
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

W13_BYTES = 2 * (2048 * 4096 // 2 + 2048 * 4096 // 32)   # gate+up codes and scales of one expert
W2_BYTES = 4096 * 2048 // 2 + 4096 * 2048 // 32
METRIC = "moe_layer_decode_tokens_per_s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tokens", type=int, default=32, help="decode tokens per GPU per step")
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--batches", type=int, default=8, help="distinct activation batches cycled")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default=None, choices=["model", "moe_layer", "fp8_gemm", "attn"],
                    help="model: full 43-layer token loop (default); moe_layer: one MoE sublayer (config 2); "
                         "fp8_gemm: the FP8 dense GEMM of config 1 (W [4096,4096], M = 1, 32, 512, 4096); "
                         "attn: sparse-attention decode over long synthetic KV caches (config 3)")
    ap.add_argument("--ctx", default="8192,131072,1048576", help="attn workload: context lengths")
    ap.add_argument("--attn-batches", default="1,32", help="attn workload: decode queries per step (per GPU)")
    ap.add_argument("--batch", type=int, default=32, help="model workload: sequences decoded in lockstep")
    ap.add_argument("--prompt", type=int, default=512, help="model workload: prompt tokens per sequence")
    ap.add_argument("--no-mtp", action="store_true", help="model workload: skip the batch-1 run with MTP speculative drafting")
    ap.add_argument("--mtp-depth", type=int, default=2, help="drafts chained per speculative step")
    ap.add_argument("--layers", type=int, default=43, help="model workload: layers (43 = the real model)")
    ap.add_argument("--microbatches", type=int, default=1,
                    help="model workload, 1 GPU: model objects the batch is split over; they share the weights "
                         "and step side by side on streams of their own")
    a = ap.parse_args()
    if a.workload is None:
        a.workload = "model"
    if a.workload == "model" and a.steps == 400 and a.warmup == 20:
        a.steps, a.warmup = 64, 4          # defaults of the token-loop workload
    return a


def workload_config(a, n):
    return {"workload": f"config2: one MoE sublayer at V4-Flash dims, decode T={a.tokens} per GPU",
            "hidden": 4096, "moe_intermediate": 2048, "n_routed_experts": a.experts, "topk": 6,
            "tokens_per_gpu": a.tokens, "global_tokens": a.tokens * n,
            "parallelism": f"ep{n}" if n > 1 else "single",
            "l2": "experts touched per step (>1 GB) exceed the 126 MB L2; activation batches cycle"}


class ClockSampler:
    """nvidia-smi clock/throttle samples during the timed region."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", uuid, f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0, t1):
        if self.proc:
            self.proc.terminate()
        rows = [r for t, r in self.rows if t0 <= t <= t1] or [r for _, r in self.rows[-3:]]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(float(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][1]), "reasons": reasons,
                "samples": len(rows)}


def peak_hbm():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---- the reference's CPU implementation (cpu_baseline and --impl reference) ---------------
def cpu_moe_runner(W, tokens):
    """Returns (callable running one T-token apus_moe_forward on the host, kind, cores)."""
    from _oracle import P, ora_moe, ref
    from apus_b200 import capi
    L = ref()
    rng = np.random.default_rng(12345)
    from apus_b200 import synth
    x = synth.activations(rng, tokens, W.dim)
    if L is not None:
        w = W.moew()
        out = np.empty((tokens, W.dim), np.float32)

        def run():
            L.apus_moe_forward(C.byref(w), P(x), None, tokens, P(out), None)
        run.keep = (w, out)
        return run, "reference", L.ref_pool_threads
    return (lambda: ora_moe(W, x)), "port", (lambda: 1)


def time_cpu(run, tokens, budget_s, min_steps=1, max_steps=10 ** 9):
    run()                                   # warm-up (spawns the pool, faults pages in)
    t0 = time.perf_counter()
    n = 0
    while n < min_steps or (time.perf_counter() - t0 < budget_s and n < max_steps):
        run()
        n += 1
    dt = time.perf_counter() - t0
    return tokens * n / dt, n, dt


def reference_arm(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    os.environ.setdefault("APUS_THREADS", str(min(os.cpu_count() or 1, 32)))
    from apus_b200 import synth
    W = synth.MoeWeights(seed=a.seed, E=a.experts)
    run, kind, cores = cpu_moe_runner(W, a.tokens)
    for _ in range(max(a.warmup, 1) if kind == "reference" else 1):
        run()
    steps = a.steps if kind == "reference" else min(a.steps, 2)
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = time.perf_counter() - t0
    val = a.tokens * steps / dt
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "tok/s", "n_gpus": a.gpus,
            "steps": steps, "warmup": a.warmup, "ms_per_step": dt / steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config(a, a.gpus),
            "cpu_baseline": {"value": val, "unit": "tok/s", "cores": cores(), "kind": kind,
                             "sample": f"{steps} steps of T={a.tokens} tokens through apus_moe_forward "
                                       f"on the host ({'unmodified reference C, AVX2 rows' if kind == 'reference' else 'oracle port'})"},
            "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


# ---- full-model token loop (config 4 of the baseline; the headline metric) ------------------
MODEL_METRIC = "decode_tokens_per_s"


def model_config(a, n, cfg, L=None):
    kinds = cfg.layer_kinds()
    return {"workload": f"config4: full DeepSeek-V4-Flash token loop, random-init weights generated on the device, "
                        f"{a.prompt}-token prompt then greedy decode at batch {a.batch}",
            "layers": cfg.n_layers, "layer_kinds": {"swa": kinds.count(0), "csa": kinds.count(4), "hca": kinds.count(128)},
            "hidden": cfg.dim, "n_routed_experts": cfg.n_experts, "topk": cfg.topk, "vocab": cfg.vocab,
            "batch": a.batch, "prompt_tokens": a.prompt, "parallelism": f"ep{n}" if n > 1 else "single",
            "microbatches": 1 if n > 1 else max(1, a.microbatches),
            "sum_order": sum_order_name(L),
            "l2": "each step streams the touched experts and all dense weights (>20 GB at batch 32), far above the 126 MB L2"}


def token_digest(L, toks):
    """64-bit FNV-1a over the int32 tokens [sequences, steps], as a hex string."""
    t = np.ascontiguousarray(toks.astype(np.int32))
    return f"{L.apus_fnv1a(t.ctypes.data, t.nbytes, 0xcbf29ce484222325):016x}"


def sum_order_name(L=None):
    if L is None:
        return "default"
    m = L.apus_cuda_set_tree_ops(-1)
    return "reference" if m == 0 else f"tree mask {m}" + (" (default)" if m == L.apus_cuda_set_tree_ops(-2) else "")


def flash_config(a):
    from apus_b200.flash import FlashConfig
    cfg = FlashConfig()
    if a.layers != cfg.n_layers:
        cfg.n_layers = a.layers
    if a.experts != cfg.n_experts:
        cfg.n_experts = a.experts
    return cfg


def mtp_arm(L, W, h, a, cfg):
    """Batch 1 with MTP speculative drafting (reference c/mtp.h:472-616): the draft head chains
    `depth` candidates, the main model verifies them in one pass, accepted ones are emitted with
    the model's own pick.  The head is random-init like the model, so it predicts nothing: the
    acceptance rate is what a random head earns, and the line shows what the machinery costs;
    the emitted stream must be the plain greedy stream either way."""
    import apus_b200
    from apus_b200 import capi
    from apus_b200.flash import prompt_ids
    depth, n_gen = a.mtp_depth, min(a.steps, 64)
    d = W.mtp_desc(0)
    mt = L.apus_cuda_mtp_create(h, C.byref(d))
    if not mt:
        apus_b200.check(1, "apus_cuda_mtp_create")
    prompt = np.ascontiguousarray(prompt_ids(a.seed, 0, 1, a.prompt, cfg.vocab))
    try:
        plain = np.zeros((1, n_gen), np.int32)
        apus_b200.check(L.apus_cuda_model_reset(h), "model_reset")
        apus_b200.check(L.apus_cuda_model_generate(h, capi.ptr(prompt), a.prompt, n_gen, capi.ptr(plain), None, None), "generate")
        toks, stats = np.zeros(n_gen, np.int32), np.zeros(8, np.uint64)
        times = []
        for n in (4, n_gen):                                  # the short run warms the head's buffers up
            apus_b200.check(L.apus_cuda_model_reset(h), "model_reset")
            t0 = time.perf_counter()
            apus_b200.check(L.apus_cuda_model_spec_generate_mtp(h, mt, capi.ptr(prompt), a.prompt, n, depth, capi.ptr(toks),
                                                                 capi.ptr(stats)), "spec_generate_mtp")
            times.append(time.perf_counter() - t0)
        # both runs consume the prompt; their difference is n_gen - 4 emitted tokens of draft/verify steps
        dt = times[1] - times[0]
        emitted = n_gen - 4
    finally:
        L.apus_cuda_mtp_destroy(mt)
    return {"value": emitted / dt if dt > 0 else None, "unit": "tok/s", "batch": 1, "depth": depth, "tokens": n_gen,
            "ms_per_token": dt / max(emitted, 1) * 1e3, "tokens_equal_plain_greedy": bool(np.array_equal(toks, plain[0])),
            "verify_batches": int(stats[1]), "batch_tokens": int(stats[2]), "refeed_tokens": int(stats[3]),
            "drafts_offered": int(stats[4]), "drafts_accepted": int(stats[5]), "d1_hits": int(stats[7]),
            "head": "random-init MTP block (sliding window, 256 experts) + e/h projections, generated on the device",
            "timing": "host clock around the loop (it synchronises every step to read the draft ids)"}


def dspark_arm(L, W, h, a, cfg):
    """Batch 1 with the DSpark draft module (reference c/dspark.h:747-862): per round a block of 5 drafts from
    three random-init stages, verified in one pass of 6 positions.  As with the MTP head a random module
    predicts nothing; the line shows the cost of a round and that the stream is the plain greedy stream."""
    import apus_b200
    from apus_b200 import capi
    from apus_b200.flash import prompt_ids
    n_gen = min(a.steps, 64)
    d = W.dspark_desc()
    ds = L.apus_cuda_dspark_create(h, C.byref(d))
    if not ds:
        apus_b200.check(1, "apus_cuda_dspark_create")
    prompt = np.ascontiguousarray(prompt_ids(a.seed, 0, 1, a.prompt, cfg.vocab))
    try:
        plain = np.zeros((1, n_gen), np.int32)
        apus_b200.check(L.apus_cuda_model_reset(h), "model_reset")
        apus_b200.check(L.apus_cuda_model_generate(h, capi.ptr(prompt), a.prompt, n_gen, capi.ptr(plain), None, None), "generate")
        toks, stats = np.zeros(n_gen, np.int32), np.zeros(7, np.uint64)
        times = []
        for n in (4, n_gen):
            apus_b200.check(L.apus_cuda_model_reset(h), "model_reset")
            t0 = time.perf_counter()
            apus_b200.check(L.apus_cuda_model_spec_generate_dspark(h, ds, capi.ptr(prompt), a.prompt, n, capi.ptr(toks),
                                                                    capi.ptr(stats)), "spec_generate_dspark")
            times.append(time.perf_counter() - t0)
        dt, emitted = times[1] - times[0], n_gen - 4
    finally:
        L.apus_cuda_dspark_destroy(ds)
    return {"value": emitted / dt if dt > 0 else None, "unit": "tok/s", "batch": 1, "block_size": int(d.block_size),
            "stages": int(d.n_stages), "tokens": n_gen, "ms_per_token": dt / max(emitted, 1) * 1e3,
            "tokens_equal_plain_greedy": bool(np.array_equal(toks, plain[0])), "verify_batches": int(stats[1]),
            "batch_tokens": int(stats[2]), "refeed_tokens": int(stats[3]), "drafts_offered": int(stats[4]),
            "drafts_accepted": int(stats[5]), "bonus_rounds": int(stats[6]),
            "module": "random-init DSpark stages + main projection + bigram / confidence heads, generated on the device "
                      "(block size, target layers and bigram rank are stand-ins)",
            "timing": "host clock around the loop"}


def cpu_model_baseline(cfg, seed, budget_s, prompt=512):
    """The reference's decode step composed from its own apus_block_forward timed
    on one layer of each kind at full size (E experts, one token per call at the
    positions the GPU arm decodes at: after a `prompt`-token prefill of that layer)
    plus the head: t = sum_kinds n_kind * t_kind + t_head.  A projection: the whole
    model (158 GB) does not fit the time budget of a benchmark run on the host."""
    import cases
    from _oracle import P, ref
    from apus_b200 import capi, synth
    from apus_b200.flash import rope_tables
    L = ref()
    if L is None:
        return None
    rng = np.random.default_rng(seed)
    dims = dict(dim=cfg.dim, n_heads=cfg.n_heads, head_dim=cfg.head_dim, rope_dim=cfg.rope_dim, q_lora=cfg.q_lora,
                o_groups=cfg.o_groups, o_lora=cfg.o_lora, window=cfg.window, idx_heads=cfg.idx_heads,
                idx_dim=cfg.idx_dim, idx_topk=cfg.idx_topk, max_pos=prompt + 64)
    mdims = dict(E=cfg.n_experts, topk=cfg.topk, inter=cfg.inter)
    L.ref_block_forward.restype = None
    L.ref_block_forward.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_float, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_int, C.c_int64]
    kinds = cfg.layer_kinds()
    t_kind, moe, calls = {}, None, 0
    for ratio, kind in ((0, "swa"), (4, "csa"), (128, "hca128")):
        if ratio not in kinds:
            continue
        cos, sin = rope_tables(cfg, ratio != 0, prompt + 64)
        B = cases.BlockLayer(seed + ratio, kind, cos, sin, dims=mdims, attn_dims=dims)
        if moe is None:
            moe = B.moe                                  # 3.4 GB of experts: generated once, shared by the kinds
        else:
            B.moe = moe
            B.desc.mw = moe.moew()
        S = cases.AttnState(B.attn)
        h = cases.block_inputs(seed + 3, prompt + 1, cfg.hc_mult, cfg.dim)
        ids = np.zeros(prompt + 1, np.int64)
        L.ref_block_forward(C.byref(B.desc), cfg.hc_mult, cfg.hc_iters, cfg.hc_eps, cfg.norm_eps, C.byref(S.st),
                            P(h[:prompt]), P(ids[:prompt]), prompt, 0)           # untimed: fills the window and the caches
        n, t0 = 0, time.perf_counter()
        while n < 3 or (time.perf_counter() - t0 < budget_s / 3 and n < 40):
            hh = h[prompt:prompt + 1].copy()
            L.ref_block_forward(C.byref(B.desc), cfg.hc_mult, cfg.hc_iters, cfg.hc_eps, cfg.norm_eps, C.byref(S.st),
                                P(hh), P(ids[prompt:prompt + 1]), 1, prompt + n)
            n += 1
        t_kind[ratio] = (time.perf_counter() - t0) / n
        calls += n
    # head: BF16 [vocab, dim] GEMV
    head = synth.bf16_bits((rng.standard_normal((cfg.vocab, cfg.dim)) * 0.02).astype(np.float32))
    x = synth.activations(rng, 1, cfg.dim)
    out = np.empty(cfg.vocab, np.float32)
    L.ref_head_gemv.restype = None
    L.ref_head_gemv.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64]
    L.ref_head_gemv(P(head), P(x), P(out), cfg.vocab, cfg.dim)
    t0 = time.perf_counter()
    n = 0
    while n < 3:
        L.ref_head_gemv(P(head), P(x), P(out), cfg.vocab, cfg.dim)     # c/model.h:638-647
        n += 1
    t_head = (time.perf_counter() - t0) / n
    t_step = sum(t_kind[r] for r in kinds) + t_head
    return {"value": 1.0 / t_step, "unit": "tok/s", "cores": L.ref_pool_threads(), "kind": "reference",
            "projected": True, "timed_calls": calls + 3,
            "sample": f"one decode token per call (positions {prompt}+, after a {prompt}-token prefill of the layer) through "
                      "the unmodified apus_block_forward at full sizes, one layer of each kind with 256 experts ("
                      + ", ".join(f"{k}: {v * 1e3:.0f} ms" for k, v in t_kind.items())
                      + f"), head GEMV {t_head * 1e3:.0f} ms; step = sum over the {cfg.n_layers} layers + head; "
                        "the reference decodes sequences one at a time, so its tok/s does not grow with the batch"}


def model_reference_arm(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    os.environ.setdefault("APUS_THREADS", str(min(os.cpu_count() or 1, 32)))
    cfg = flash_config(a)
    cb = cpu_model_baseline(cfg, a.seed, budget_s=20.0, prompt=a.prompt)
    if cb is None:
        emit({"impl": "reference", "unavailable": "the reference build (oracle/_ref) is not present"})
        return
    import apus_b200
    # `steps` = the block calls actually timed (the step time is composed from them, see cpu_baseline.sample)
    line = {"impl": "reference", "metric": MODEL_METRIC, "value": cb["value"], "unit": "tok/s", "n_gpus": a.gpus,
            "steps": cb["timed_calls"], "warmup": 1, "ms_per_step": 1e3 / cb["value"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "projected": True,
            "config": model_config(a, a.gpus, cfg, apus_b200.lib()), "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


def model_main_ep(a):
    """N > 1: every rank decodes its own batch; the routed experts are sharded over
    the ranks and token rows travel by NCCL all-to-all inside every layer."""
    import datetime
    import torch
    import torch.distributed as dist
    import apus_b200
    from apus_b200.ep_model import EpModel
    from apus_b200.flash import RandomFlashModel
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == a.gpus, f"--gpus {a.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if "MASTER_ADDR" not in os.environ:                   # single process (one-rank test of this loop)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29533", RANK="0", WORLD_SIZE="1")
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=60))
    apus_b200.build()
    L = apus_b200.lib()
    err = C.create_string_buffer(512)
    if L.apus_cuda_enable(err, 512):
        raise RuntimeError(err.value.decode())
    cfg = flash_config(a)
    B, K, Wm = a.batch, a.steps, a.warmup
    per = cfg.n_experts // world
    max_pos = a.prompt + 2 * (K + Wm) + 80
    W = RandomFlashModel(cfg, a.seed, dev, e_lo=rank * per, e_hi=(rank + 1) * per, max_pos=max_pos)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    ep = EpModel(W.desc, cfg.n_layers, cfg.n_experts, cfg.topk, cfg.dim, B, max_pos, rank, world, device=dev)
    from apus_b200.flash import prompt_ids
    # sequence g of the job (rank r holds g = r*B ..) has the prompt of sequence g of a one-GPU run
    prompt = prompt_ids(a.seed, rank * B, B, a.prompt, cfg.vocab)
    hist = torch.zeros(Wm + K + 3, B, dtype=torch.int64, device=dev)      # the token every step picked
    n_hist = [0]

    def keep_tokens():
        hist[n_hist[0]].copy_(ep.ids)                  # the pick was fed back into the ids on the device
        n_hist[0] += 1
    uuid = str(torch.cuda.get_device_properties(dev).uuid)
    sampler = ClockSampler(uuid if uuid.startswith("GPU-") else "GPU-" + uuid) if rank == 0 else None

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()
    def mark(msg):
        if os.environ.get("APUS_BENCH_TRACE"):
            print(f"[rank {rank}] {msg}", file=sys.stderr, flush=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    mark("prefill")
    e0.record()
    ep.prefill(prompt)
    e1.record()
    torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1)
    keep_tokens()
    mark("warm-up steps")
    for _ in range(Wm):
        ep.step()
        keep_tokens()
    torch.cuda.synchronize()
    mark("warm-up done")
    d0 = L.apus_cuda_dispatches()
    recorded, ep.graph = ep.graph, None                 # the prompt may have left a recorded step behind
    ep.step()
    ep.graph = recorded
    keep_tokens()
    per_step = int(L.apus_cuda_dispatches() - d0)       # kernels of one step, counted on plain launches
    graph_note = "each step replayed from one CUDA graph (library kernels + NCCL all-to-alls)"
    if os.environ.get("APUS_EP_GRAPH", "1") != "0":
        try:
            if not ep.graph:
                ep.capture()
        except Exception as e:                          # keep going on plain launches
            graph_note = f"plain launches (graph capture failed: {type(e).__name__}: {e})"
            torch.cuda.synchronize()
    else:
        graph_note = "plain launches"
    mark(graph_note)
    ep.step()
    keep_tokens()
    barrier()
    mark("timed region")
    w0 = time.time()
    e0.record()
    for _ in range(K):
        ep.step()
        keep_tokens()
    e1.record()
    barrier()
    w1 = time.time()
    digest = token_digest(L, hist[:Wm + K + 2].t().cpu().numpy()) if rank == 0 else None
    launches = per_step * K
    tms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms = float(tms.item())
    clocks = sampler.stop(w0, w1) if sampler else None
    # end to end: ids from the host, sampled ids back to the host, every step
    nxt = np.empty(B, np.int32)
    ep.read(tokens=nxt)
    ne = max(8, K // 4)
    barrier()
    t0 = time.perf_counter()
    for _ in range(ne):
        ep.set_ids(nxt.astype(np.int64))
        ep.step()                            # the recorded step; its own feed-back is overwritten by the next set_ids
        ep.read(tokens=nxt)
    barrier()
    te = torch.tensor([time.perf_counter() - t0], device=dev)
    dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_val = world * B * ne / float(te.item())
    ep.graph = None
    ep.close()

    # ---- fixed total batch (strong scaling): `gb` sequences over all ranks; at gb = 1 every rank steps
    # the same single sequence (the dense path is replicated and deterministic), its routed experts
    # still live on their owners, so dispatch and combine cross the links as they would
    def strong(gb):
        per_rank = max(1, gb // world)
        first = rank * per_rank if gb >= world else 0
        m2 = EpModel(W.desc, cfg.n_layers, cfg.n_experts, cfg.topk, cfg.dim, per_rank, max_pos, rank, world, device=dev)
        try:
            m2.prefill(prompt_ids(a.seed, first, per_rank, min(a.prompt, 16), cfg.vocab))
            for _ in range(2):
                m2.step()
            if os.environ.get("APUS_EP_GRAPH", "1") != "0":
                try:
                    m2.capture()
                except Exception:
                    torch.cuda.synchronize()
            m2.step()
            barrier()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ks = max(8, K // 2)
            s0.record()
            for _ in range(ks):
                m2.step()
            s1.record()
            barrier()
            t = torch.tensor([s0.elapsed_time(s1)], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            seqs = gb if gb >= world else 1
            return {"global_batch": seqs, "per_rank": per_rank, "steps": ks, "ms_per_step": float(t.item()) / ks,
                    "value": seqs * ks / (float(t.item()) * 1e-3), "unit": "tok/s", "prompt_tokens": min(a.prompt, 16)}
        finally:
            m2.graph = None
            m2.close()
    strong32 = strong(32) if world <= 32 else None
    strong1 = strong(1)
    if rank == 0:
        line = {
            "metric": MODEL_METRIC, "value": world * B * K / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": K, "warmup": Wm, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f32 accumulate over E2M1xE4M3 / E4M3xE4M3 tensor-core products; BF16-valued activations",
            "data": "synthetic", "config": model_config(a, world, cfg, L), "clocks": clocks,
            "e2e": {"value": e2e_val, "unit": "tok/s", "h2d_bytes_per_step": world * B * 8,
                    "d2h_bytes_per_step": world * B * 4, "steps": ne},
            "gpu_launches": launches,
            "tokens_fnv1a": digest, "digest_tokens_per_seq": Wm + K + 2,
            "strong_bs32": strong32, "strong_bs1": strong1,
            "prefill": {"tokens": world * B * a.prompt, "ms": prefill_ms,
                        "note": "expert-parallel loop: prompt consumed as consecutive decode steps replayed from the recorded step"},
            "roofline": None, "weights": {"bytes_per_rank": W.bytes}, "cuda_graph": graph_note,
            "note": "expert-parallel: experts sharded over the ranks, NCCL all-to-all dispatch/combine per layer; "
                    "the per-kernel roofline is reported by the 1-GPU run"}
        emit(line)
    # captured graphs held NCCL work; leave without tearing the communicator down
    # (destroying the group with such graphs alive can block)
    barrier()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def model_main(a):
    # APUS_EP_TEST=1: run the expert-parallel loop (padded exchange, graph capture) with one rank
    if a.gpus > 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1 or os.environ.get("APUS_EP_TEST") == "1":
        return model_main_ep(a)
    import torch
    import apus_b200
    from apus_b200 import capi
    from apus_b200.flash import RandomFlashModel
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    apus_b200.build()
    L = apus_b200.lib()
    err = C.create_string_buffer(512)
    if L.apus_cuda_enable(err, 512):
        raise RuntimeError(err.value.decode())
    cfg = flash_config(a)
    B, K, Wm = a.batch, a.steps, a.warmup
    max_pos = a.prompt + 2 * (K + Wm) + 72
    t0 = time.time()
    W = RandomFlashModel(cfg, a.seed, dev, max_pos=max_pos)
    torch.cuda.synchronize()
    t_gen = time.time() - t0
    torch.cuda.empty_cache()

    def create(batch):
        h = L.apus_cuda_model_create(C.byref(W.desc), batch, max_pos)
        if not h:
            apus_b200.check(1, "apus_cuda_model_create")
        return h
    from apus_b200.flash import prompt_ids
    uuid = str(torch.cuda.get_device_properties(dev).uuid)
    sampler = ClockSampler(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)

    def parr(arrays):
        return (C.c_void_p * len(arrays))(*[capi.ptr(x) for x in arrays])

    def run(batch, groups):
        """`batch` sequences held by `groups` model objects (batch / groups each) that share
        the device-resident weights and step side by side, each on its own stream.
        Prompt, warm-up decode steps, K timed decode steps with the sampled token fed back
        on the device (each model's step replayed from its CUDA graph); then a short pass
        of the first model alone with plain launches and CUDA events around the expert
        kernels.  Returns (handles, ms of the K steps, prefill ms, kernels in the timed
        region, last tokens per model, wall, stats)."""
        per = batch // groups
        hs = [create(per) for _ in range(groups)]
        if groups > 1:
            for h in hs:
                apus_b200.check(L.apus_cuda_model_set_stream(h, None, 1), "model_set_stream")
        harr = (C.c_void_p * groups)(*hs)
        prompts = [np.ascontiguousarray(prompt_ids(a.seed, g * per, per, a.prompt, cfg.vocab)) for g in range(groups)]
        toks = [np.empty((per, Wm + 1), np.int32) for _ in range(groups)]
        ms_pre, ms_dec = C.c_float(0), C.c_float(0)
        apus_b200.check(L.apus_cuda_model_generate_group(harr, groups, parr(prompts), a.prompt, Wm + 1, parr(toks),
                                                         C.byref(ms_pre), C.byref(ms_dec)),
                        "generate (prompt + warm-up)")
        prefill_ms = ms_pre.value
        last = [np.ascontiguousarray(t[:, -1:].astype(np.int64)) for t in toks]
        out = [np.empty((per, K + 1), np.int32) for _ in range(groups)]
        torch.cuda.synchronize()
        w0 = time.time()
        apus_b200.check(L.apus_cuda_model_generate_group(harr, groups, parr(last), 1, K + 1, parr(out),
                                                         C.byref(ms_pre), C.byref(ms_dec)), "generate (timed)")
        torch.cuda.synchronize()
        w1 = time.time()
        ms = ms_dec.value
        # plain-launch pass of the first model alone: kernels per step, and events around the expert GEMVs
        h = hs[0]
        moes = [L.apus_cuda_model_moe(h, i) for i in range(cfg.n_layers)]
        kt = min(K, 16)
        for m in moes:
            L.apus_cuda_moe_timing(m, 1)
            L.apus_cuda_moe_work_items(m, 1)
        last0 = np.ascontiguousarray(out[0][:, -1:].astype(np.int64))
        out2 = np.empty((per, kt + 1), np.int32)
        d0 = L.apus_cuda_dispatches()
        apus_b200.check(L.apus_cuda_model_generate(h, capi.ptr(last0), 1, kt + 1, capi.ptr(out2), C.byref(ms_pre),
                                                   C.byref(ms_dec)), "generate (event pass)")
        per_step = (int(L.apus_cuda_dispatches() - d0)) // (kt + 1)
        ms_plain = ms_dec.value / kt
        g13 = g2 = 0.0
        nl = items = 0
        for m in moes:
            x, y, n = C.c_double(), C.c_double(), C.c_int()
            apus_b200.check(L.apus_cuda_moe_timing_read(m, C.byref(x), C.byref(y), C.byref(n)), "timing")
            L.apus_cuda_moe_timing(m, 0)
            g13 += x.value; g2 += y.value; nl += n.value
            items += L.apus_cuda_moe_work_items(m, 0)
        stats = (g13, g2, nl, items, kt, ms_plain)
        stream_toks = [np.concatenate([toks[g], out[g]], axis=1) for g in range(groups)]   # t0 .. t(Wm+K+1) per sequence
        # the other models catch up with the first one's event pass (same position for the e2e loop)
        for g in range(1, groups):
            lg = np.ascontiguousarray(out[g][:, -1:].astype(np.int64))
            o2 = np.empty((per, kt + 1), np.int32)
            apus_b200.check(L.apus_cuda_model_generate(hs[g], capi.ptr(lg), 1, kt + 1, capi.ptr(o2), None, None),
                            "generate (catch up)")
            out[g] = o2
        out[0] = out2
        return hs, ms, prefill_ms, per_step * K * groups, out, (w0, w1), stats, np.concatenate(stream_toks, axis=0)

    G = max(1, a.microbatches)
    if B % G:
        raise SystemExit(f"--batch {B} is not a multiple of --microbatches {G}")
    hs, ms, prefill_ms, launches, out, wall, stats, stream = run(B, G)
    digest = token_digest(L, stream[:, :Wm + K + 2])
    clocks = sampler.stop(*wall)
    value = B * K / (ms * 1e-3)

    # ---- end to end: ids from the host every step, sampled ids back to the host -----------------
    per = B // G
    harr = (C.c_void_p * G)(*hs)
    ids = [np.ascontiguousarray(o[:, -1:].astype(np.int64)) for o in out]
    nxt = [np.empty(per, np.int32) for _ in range(G)]
    ne = max(8, K // 4)

    def e2e_step():
        apus_b200.check(L.apus_cuda_model_forward_group(harr, G, parr(ids), 1, None, parr(nxt)), "model_forward")
        for g in range(G):
            ids[g][:, 0] = nxt[g]
    for _ in range(3):
        e2e_step()
    t0 = time.perf_counter()
    for _ in range(ne):
        e2e_step()
    e2e_val = B * ne / (time.perf_counter() - t0)
    for h in hs:
        L.apus_cuda_model_destroy(h)

    # ---- batch 1 ------------------------------------------------------------------------------
    h1, ms1, prefill1, launches1, out1, _, st1, stream1 = run(1, 1)
    mtp_line = dspark_line = None
    if not a.no_mtp:
        mk = W.mark()
        mtp_line = mtp_arm(L, W, h1[0], a, cfg)
        W.drop(mk)
        dspark_line = dspark_arm(L, W, h1[0], a, cfg)
        W.drop(mk)
    L.apus_cuda_model_destroy(h1[0])

    peak, peak_kind = peak_hbm()
    g13, g2, nl, items, kt, ms_plain = stats
    ms_ev = ms_plain * (kt + 1)                  # time of the event pass, for the kernels' share of a step
    achieved = items * W13_BYTES / (g13 * 1e-3) / 1e9 if g13 > 0 else None
    achieved2 = items * W2_BYTES / (g2 * 1e-3) / 1e9 if g2 > 0 else None
    line = {
        "metric": MODEL_METRIC, "value": value, "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": Wm,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 accumulate over E2M1xE4M3 / E4M3xE4M3 tensor-core products; BF16-valued activations",
        "data": "synthetic", "config": model_config(a, 1, cfg, L), "clocks": clocks,
        "e2e": {"value": e2e_val, "unit": "tok/s", "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * 4,
                "steps": ne},
        "gpu_launches": launches,
        "tokens_fnv1a": digest, "digest_tokens_per_seq": Wm + K + 2,
        "batch1": {"value": 1 * K / (ms1 * 1e-3), "unit": "tok/s", "ms_per_step": ms1 / K,
                   "gpu_launches": launches1, "prefill_ms": prefill1, "ms_per_step_plain_launches": st1[5],
                   # the expert gate/up GEMV at batch 1: 6 experts per launch, same accounting as `roofline`
                   "roofline": {"kernel": "gemm_tc_kernel<pair> at batch 1", "bound": "hbm",
                                "achieved": st1[3] * W13_BYTES / (st1[0] * 1e-3) / 1e9 if st1[0] > 0 else None,
                                "peak": peak, "unit": "GB/s",
                                "frac": st1[3] * W13_BYTES / (st1[0] * 1e-3) / 1e9 / peak if st1[0] > 0 else None,
                                "avg_launch_us": st1[0] / max(st1[2], 1) * 1e3, "avg_unique_experts": st1[3] / max(st1[2], 1),
                                "down_proj_frac": st1[3] * W2_BYTES / (st1[1] * 1e-3) / 1e9 / peak if st1[1] > 0 else None}},
        "mtp": mtp_line,
        "dspark": dspark_line,
        "prefill": {"tokens": B * a.prompt, "ms": prefill_ms, "tok_s": B * a.prompt / (prefill_ms * 1e-3),
                    "note": "prompt consumed in chunks of positions (2048 rows = positions x sequences per pass)"},
        "weights": {"bytes": W.bytes, "generate_s": t_gen},
        "roofline": {"kernel": "gemm_tc_kernel<pair> (tcgen05 block-scaled MXFP4 expert gate/up GEMV + SwiGLU), "
                               "all layers of the timed steps",
                     "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": (achieved / peak) if achieved else None, "peak_kind": peak_kind,
                     # dram read+write bytes per launch: measured with ncu on a 64-expert case of the same
                     # kernel (1.002 x the algorithmic bytes) and scaled by the experts touched here
                     "traffic": items / max(nl, 1) * W13_BYTES * 1.002,
                     "traffic_source": "ncu capture of a smaller case scaled by units (profiles/gemm_tc_mxfp4_pair_T32_E64.md)",
                     "launches": nl, "avg_launch_us": g13 / max(nl, 1) * 1e3,
                     "avg_unique_experts": items / max(nl, 1),
                     "share_of_step": g13 / ms_ev if ms_ev > 0 else None,
                     "events": f"CUDA events around every launch in a pass of {kt} plain-launch steps right after the "
                               "timed region (a replayed graph cannot carry readable events)",
                     "down_proj_kernel": {"achieved": achieved2, "frac": (achieved2 / peak) if achieved2 else None,
                                          "avg_launch_us": g2 / max(nl, 1) * 1e3, "share_of_step": g2 / ms_ev}},
        "cuda_graph": {"replayed_steps": K, "ms_per_step_plain_launches": ms_plain},
    }
    if not a.no_cpu_baseline:
        os.environ.setdefault("APUS_THREADS", str(min(os.cpu_count() or 1, 32)))
        cb = cpu_model_baseline(cfg, a.seed, budget_s=20.0, prompt=a.prompt)
        if cb:
            line["cpu_baseline"] = cb
    emit(line)


# ---- config 1: FP8 E4M3 block-scaled dense GEMM ------------------------------------------------
def fp8_gemm_main(a):
    """W [4096, 4096] E4M3 with 128x128 UE8M0 tile scales, activations [M, 4096] quantised per
    token per 128 (act quant + tcgen05 kernel + BF16 round = apus_fp8_linear), device resident."""
    import torch
    import apus_b200
    from apus_b200 import capi, synth
    torch.cuda.set_device(0)
    apus_b200.build()
    L = apus_b200.lib()
    err = C.create_string_buffer(512)
    if L.apus_cuda_enable(err, 512):
        raise RuntimeError(err.value.decode())
    O = K = 4096
    rng = np.random.default_rng(a.seed)
    codes, scales = synth.fp8_weight(rng, O, K)
    qw = capi.qw(codes, scales, O, K)
    h = L.apus_cuda_fp8_upload(C.byref(qw))
    if not h:
        apus_b200.check(1, "fp8_upload")
    peak, peak_kind = peak_hbm()
    res = {}
    stream = torch.cuda.current_stream().cuda_stream
    for M in (1, 32, 512, 4096):
        x = torch.from_numpy(synth.activations(rng, M, K)).cuda()
        out = torch.empty(M, O, device="cuda")
        for _ in range(max(a.warmup, 3)):
            apus_b200.check(L.apus_cuda_fp8_linear_dev(h, x.data_ptr(), out.data_ptr(), M, stream), "fp8_linear_dev")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        tot = 0.0
        n = min(a.steps, 50)
        for _ in range(n):
            flush.zero_()                                  # 256 MB write: evicts the 126 MB L2
            e0.record()
            apus_b200.check(L.apus_cuda_fp8_linear_dev(h, x.data_ptr(), out.data_ptr(), M, stream), "fp8_linear_dev")
            e1.record()
            e1.synchronize()
            tot += e0.elapsed_time(e1)
        us = tot / n * 1e3
        res[str(M)] = {"us": us, "weight_GBs": (O * K + (O // 128) * (K // 128)) / us / 1e3,
                       "TFLOPs": 2.0 * M * O * K / us / 1e6}
    line = {"metric": "fp8_dense_gemm_us", "workload": "config1: FP8 E4M3 block-scaled GEMM, W [4096,4096]",
            "n_gpus": 1, "results_by_M": res, "hbm_peak_GBs": peak, "peak_kind": peak_kind,
            "note": "act quant + gemm_tc8_kernel + BF16 round per call; L2 flushed between timed calls; "
                    "M <= 63 runs as 32-row work items, M >= 64 on the 128-rows-per-CTA kernel"}
    emit(line)


# ---- config 3: sparse-attention decode step over a long synthetic KV cache -----------------------
ATTN_H, ATTN_D, ATTN_WIN, ATTN_TOPK = 64, 512, 128, 512


def attn_case_host(seed, kind, ctx, b, nb_cap=None):
    """Inputs of one sequence of the config-3 case on the host (generator keys per sequence):
    q [64,512] BF16-valued f32, sink [64], window ring [128,512] and compressed cache [nb,512]
    as BF16 bits, indexer scores [nb] (CSA)."""
    import apus_b200
    L = apus_b200.lib()
    ratio = 4 if kind == "csa" else 128
    nb = ctx // ratio

    def fill(tid, n, k, a_, b_, dt):
        out = np.empty(n, dt)
        apus_b200.check(L.apus_synth_fill_host(out.ctypes.data, k, n, L.apus_synth_key(seed, 3000 + ratio, tid, b), a_, b_, 0), "fill")
        return out
    return dict(q=fill(1, ATTN_H * ATTN_D, 3, 0.0, 1.0, np.float32).reshape(ATTN_H, ATTN_D),
                sink=fill(2, ATTN_H, 2, 0.0, 0.5, np.float32),
                ring=fill(3, ATTN_WIN * ATTN_D, 4, 0.0, 1.0, np.uint16).reshape(ATTN_WIN, ATTN_D),
                cache=fill(4, nb * ATTN_D, 4, 0.0, 1.0, np.uint16).reshape(nb, ATTN_D),
                scores=fill(5, nb, 2, 0.0, 1.0, np.float32) if kind == "csa" else None, nb=nb, ratio=ratio)


class AttnDecodeCase:
    """Device-resident config-3 case: B sequences, each with its own ring and compressed cache
    (same generator keys as attn_case_host), and one decode step = top-512 selection over the
    indexer scores (CSA; HCA attends every entry) + index row + gathered attention."""

    def __init__(self, L, seed, kind, ctx, B, dev, first_seq=0):
        import torch
        import apus_b200
        self.L, self.kind, self.B, self.dev = L, kind, B, dev
        ratio = 4 if kind == "csa" else 128
        nb = ctx // ratio
        self.nb, self.ratio = nb, ratio
        st = torch.cuda.current_stream().cuda_stream
        f32, i16 = torch.float32, torch.int16
        self.q = torch.empty(B, ATTN_H, ATTN_D, dtype=f32, device=dev)
        self.sink = torch.empty(ATTN_H, dtype=f32, device=dev)
        self.ring = torch.empty(B, ATTN_WIN, ATTN_D, dtype=i16, device=dev)
        self.cache = torch.empty(B, nb, ATTN_D, dtype=i16, device=dev)
        self.scores = torch.empty(B, nb, dtype=f32, device=dev) if kind == "csa" else None
        key = lambda tid, b: L.apus_synth_key(seed, 3000 + ratio, tid, first_seq + b)
        for b in range(B):
            for t, tid, k, a_, b_ in ((self.q[b], 1, 3, 0.0, 1.0), (self.ring[b], 3, 4, 0.0, 1.0), (self.cache[b], 4, 4, 0.0, 1.0)):
                apus_b200.check(L.apus_synth_fill_dev(t.data_ptr(), k, t.numel(), key(tid, b), a_, b_, st), "fill")
            if self.scores is not None:
                apus_b200.check(L.apus_synth_fill_dev(self.scores[b].data_ptr(), 2, nb, key(5, b), 0.0, 1.0, st), "fill")
        apus_b200.check(L.apus_synth_fill_dev(self.sink.data_ptr(), 2, ATTN_H, L.apus_synth_key(seed, 3000 + ratio, 2, first_seq), 0.0, 0.5, st), "fill")
        self.k = min(ATTN_TOPK, nb) if kind == "csa" else nb
        self.idxw = ATTN_WIN + self.k
        self.idx = torch.empty(B, self.idxw, dtype=torch.int32, device=dev)
        self.idx[:, :ATTN_WIN] = torch.arange(ATTN_WIN, dtype=torch.int32, device=dev)      # a full window, ring order 0..127
        if kind != "csa":
            self.idx[:, ATTN_WIN:] = ATTN_WIN + torch.arange(nb, dtype=torch.int32, device=dev)
        self.topk = torch.empty(B, self.k, dtype=torch.int32, device=dev) if kind == "csa" else None
        self.o = torch.empty(B, ATTN_H, ATTN_D, dtype=f32, device=dev)
        torch.cuda.synchronize()

    def step(self):
        import torch
        import apus_b200
        L, st = self.L, torch.cuda.current_stream().cuda_stream
        if self.kind == "csa":
            apus_b200.check(L.apus_cuda_topk_stable_dev(self.scores.data_ptr(), self.nb, self.k, self.topk.data_ptr(), self.B, st), "topk")
            torch.add(self.topk, ATTN_WIN, out=self.idx[:, ATTN_WIN:])
        apus_b200.check(L.apus_cuda_sparse_attn_batch_dev(self.q.data_ptr(), self.sink.data_ptr(), ATTN_H, ATTN_D, self.idx.data_ptr(),
                                                          self.idxw, self.B, ATTN_D ** -0.5, self.ring.data_ptr(), ATTN_WIN, ATTN_WIN,
                                                          self.cache.data_ptr(), self.nb, self.nb, self.o.data_ptr(), st), "sparse_attn")

    def bytes_per_query(self):
        """Algorithmic bytes of one query: the scan of its score row (CSA) + the gathered KV rows (BF16)."""
        return (self.nb * 4 if self.kind == "csa" else 0) + self.idxw * ATTN_D * 2


def attn_reference_query(Lr, c, kind):
    """One query of the case through the reference: apus_topk_stable (c/attn.h:668) + window ids, then
    apus_sparse_attn (c/attn.h:1308) on f32 copies of the BF16 caches."""
    from _oracle import P
    widen = lambda u: (u.astype(np.uint32) << 16).view(np.float32)
    ring, cache = widen(c["ring"]), widen(c["cache"])
    nb = c["nb"]
    k = min(ATTN_TOPK, nb) if kind == "csa" else nb
    idx = np.empty(ATTN_WIN + k, np.int32)
    idx[:ATTN_WIN] = np.arange(ATTN_WIN)
    if kind == "csa":
        top = np.empty(k, np.int32)
        Lr.apus_topk_stable(P(c["scores"]), nb, k, P(top))
        idx[ATTN_WIN:] = top + ATTN_WIN
    else:
        idx[ATTN_WIN:] = ATTN_WIN + np.arange(nb)
    o = np.empty((ATTN_H, ATTN_D), np.float32)
    Lr.ref_sparse_attn(P(c["q"]), P(c["sink"]), ATTN_H, ATTN_D, P(idx), len(idx), 1, ATTN_D ** -0.5, P(ring), ATTN_WIN, P(cache), P(o))
    return o, idx


def attn_main(a):
    import torch
    import apus_b200
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    apus_b200.build()
    L = apus_b200.lib()
    err = C.create_string_buffer(512)
    if L.apus_cuda_enable(err, 512):
        raise RuntimeError(err.value.decode())
    peak, peak_kind = peak_hbm()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    res = {}
    n_it = max(3, min(a.steps, 20))
    for kind in ("csa", "hca"):
        for ctx in [int(x) for x in a.ctx.split(",")]:
            for B in [int(x) for x in a.attn_batches.split(",")]:
                case = AttnDecodeCase(L, a.seed, kind, ctx, B, dev, first_seq=rank * B)
                for _ in range(max(a.warmup, 3)):
                    case.step()
                torch.cuda.synchronize()
                # the step's five launches replayed from a CUDA graph, so that the events time the GPU
                # and not the host's launch calls (a decode loop issues them from a graph as well)
                side = torch.cuda.Stream(device=dev)
                side.wait_stream(torch.cuda.current_stream())
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    case.step()
                torch.cuda.current_stream().wait_stream(side)
                graph.replay()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                tot = 0.0
                for _ in range(n_it):
                    flush.zero_()                                  # 256 MB write: evicts the 126 MB L2
                    e0.record()
                    graph.replay()
                    e1.record()
                    e1.synchronize()
                    tot += e0.elapsed_time(e1)
                ms = tot / n_it
                if world > 1:
                    t = torch.tensor([ms], device=dev)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    ms = float(t.item())
                gbs = case.bytes_per_query() * B / (ms * 1e-3) / 1e9
                res[f"{kind}_ctx{ctx}_B{B}"] = {"us_per_step": ms * 1e3, "queries_per_s": world * B / (ms * 1e-3),
                                                "bytes_per_query": case.bytes_per_query(), "achieved_GBs_per_gpu": gbs,
                                                "frac_of_hbm": gbs / peak, "kv_rows_per_query": case.idxw}
                del graph, case
                torch.cuda.empty_cache()
    if rank != 0:
        return
    key = f"csa_ctx{a.ctx.split(',')[-1]}_B{a.attn_batches.split(',')[-1]}"
    line = {"metric": "sparse_attn_decode_queries_per_s", "value": res[key]["queries_per_s"], "unit": "queries/s",
            "n_gpus": world, "steps": n_it, "warmup": max(a.warmup, 3), "ms_per_step": res[key]["us_per_step"] / 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 accumulate over BF16 KV",
            "data": "synthetic",
            "config": {"workload": "config3: sparse-attention decode step (stable top-512 of the indexer scores + gathered "
                                   "attention over window ++ compressed cache; HCA attends every compressed entry), "
                                   "per-sequence BF16 caches", "headline_case": key, "heads": ATTN_H, "head_dim": ATTN_D,
                       "window": ATTN_WIN, "topk": ATTN_TOPK, "parallelism": f"batch split, {world} GPUs, no collective",
                       "l2": "256 MB written between timed steps"},
            "results": res, "hbm_peak_GBs": peak, "peak_kind": peak_kind,
            "roofline": {"kernel": "topk_stable_kernel + sparse_scores_kernel + sparse_pv_kernel (one decode step)",
                         "bound": "hbm", "achieved": res[key]["achieved_GBs_per_gpu"], "peak": peak, "unit": "GB/s",
                         "frac": res[key]["frac_of_hbm"], "traffic": None}}
    if not a.no_cpu_baseline:
        from _oracle import ref
        Lr = ref()
        if Lr is not None:
            ctx = int(a.ctx.split(",")[-1])
            c = attn_case_host(a.seed, "csa", ctx, 0)
            attn_reference_query(Lr, c, "csa")
            t0, n = time.perf_counter(), 0
            while n < 2 or (time.perf_counter() - t0 < 10.0 and n < 50):
                attn_reference_query(Lr, c, "csa")
                n += 1
            dt = (time.perf_counter() - t0) / n
            line["cpu_baseline"] = {"value": 1.0 / dt, "unit": "queries/s", "cores": Lr.ref_pool_threads(), "kind": "reference",
                                    "sample": f"{n} CSA queries at context {ctx}: apus_topk_stable + apus_sparse_attn on the host"}
    emit(line)


# ---- this repository's arm (one MoE sublayer) --------------------------------------------------
_RESULT_OUT = None


def emit(line):
    """The one JSON line of a run, on the process's original stdout."""
    out = _RESULT_OUT or sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    # stdout carries exactly one JSON line: keep the original descriptor for it and point
    # descriptor 1 at stderr, so that whatever a library prints (NCCL's version banner,
    # compiler notes) cannot land in front of the result
    global _RESULT_OUT
    a = parse()
    sys.stdout.flush()
    _RESULT_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if a.workload == "fp8_gemm":
        return fp8_gemm_main(a)
    if a.workload == "attn":
        return attn_main(a)
    if a.workload == "model":
        return model_reference_arm(a) if a.impl == "reference" else model_main(a)
    if a.impl == "reference":
        return reference_arm(a)
    import torch
    import torch.distributed as dist
    import apus_b200
    from apus_b200 import capi, synth
    from apus_b200.moe import ExpertParallelMoe, create_handle

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=torch.device("cuda", local),
                                timeout=datetime.timedelta(seconds=90))
    assert world == a.gpus, f"--gpus {a.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    apus_b200.build()
    L = apus_b200.lib()
    err = C.create_string_buffer(512)
    if L.apus_cuda_enable(err, 512):
        raise RuntimeError(err.value.decode())

    T, E, K, Wm = a.tokens, a.experts, a.steps, a.warmup
    n_local = E // world
    W = synth.MoeWeights(seed=a.seed, E=E, e_lo=rank * n_local, e_hi=(rank + 1) * n_local)
    moew = W.moew()
    if world == 1:
        handle = L.apus_cuda_moe_get(C.byref(moew))
        if not handle:
            apus_b200.check(1, "apus_cuda_moe_get")
    else:
        handle = create_handle(moew, W.e_lo, W.e_hi)
    ep = ExpertParallelMoe(E, W.topk, W.dim, rank, world, handle=handle)

    rng = np.random.default_rng([a.seed, 777, rank])
    host_x = [torch.from_numpy(synth.activations(rng, T, W.dim)).pin_memory() for _ in range(a.batches)]
    dev_x = [h.to(dev) for h in host_x]
    dev_out = torch.empty(T, W.dim, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    def step_dev(b):
        if world == 1:
            apus_b200.check(L.apus_cuda_moe_forward_dev(handle, dev_x[b].data_ptr(), None, T,
                                                        dev_out.data_ptr(), stream), "moe_forward_dev")
            return dev_out
        return ep.forward(dev_x[b])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # unique local experts touched per batch (for the algorithmic bytes of the GEMV kernels)
    uniq = []
    for b in range(a.batches):
        step_dev(b)
        torch.cuda.synchronize()
        if world == 1:
            idx = np.empty((T, W.topk), np.int32)
            wg = np.empty((T, W.topk), np.float32)
            apus_b200.check(L.apus_cuda_moe_last_routing(handle, T, capi.ptr(idx), capi.ptr(wg), stream),
                            "last_routing")
            uniq.append(len(np.unique(idx)))
        else:
            idx, _ = ep.route_fn(dev_x[b], None)
            allidx = [torch.empty_like(idx) for _ in range(world)]
            dist.all_gather(allidx, idx)
            flat = torch.cat(allidx).reshape(-1)
            mine = flat[(flat >= W.e_lo) & (flat < W.e_hi)]
            uniq.append(int(torch.unique(mine).numel()))
    uuid = str(torch.cuda.get_device_properties(dev).uuid)
    sampler = ClockSampler(uuid if uuid.startswith("GPU-") else "GPU-" + uuid) if rank == 0 else None
    for i in range(Wm):
        step_dev(i % a.batches)
    barrier()
    t_spin = time.time()                       # give the sampler time to come up (untimed)
    while sampler and not sampler.rows and time.time() - t_spin < 3.0:
        time.sleep(0.02)                       # rank-local wait: no collective in here
    L.apus_cuda_moe_timing(handle, 1)
    d0 = L.apus_cuda_dispatches()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_wall0 = time.time()
    ev0.record()
    for i in range(K):
        step_dev(i % a.batches)
    ev1.record()
    barrier()
    t_wall1 = time.time()
    ms = ev0.elapsed_time(ev1)
    launches = int(L.apus_cuda_dispatches() - d0)
    g13, g2, nl = C.c_double(), C.c_double(), C.c_int()
    apus_b200.check(L.apus_cuda_moe_timing_read(handle, C.byref(g13), C.byref(g2), C.byref(nl)), "timing")
    L.apus_cuda_moe_timing(handle, 0)
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None
    if world > 1:
        tms = torch.tensor([ms], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = float(tms.item())
    value = world * T * K / (ms * 1e-3)

    # ---- end to end through host buffers -------------------------------------------------
    host_out = torch.empty(T, W.dim).pin_memory()

    def step_e2e(b):
        if world == 1:
            apus_b200.check(L.apus_cuda_moe_forward(C.byref(moew), host_x[b].data_ptr(), None, T,
                                                    host_out.data_ptr(), None), "moe_forward")
        else:
            x = host_x[b].to(dev, non_blocking=True)
            host_out.copy_(ep.forward(x), non_blocking=True)
            torch.cuda.synchronize()
    for i in range(max(3, Wm)):
        step_e2e(i % a.batches)
    barrier()
    t0 = time.perf_counter()
    for i in range(K):
        step_e2e(i % a.batches)
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        te = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_s = float(te.item())
    e2e_val = world * T * K / e2e_s

    if rank == 0:
        peak, peak_kind = peak_hbm()
        steps_uniq = [uniq[i % a.batches] for i in range(K)]
        bytes13 = float(sum(steps_uniq)) * W13_BYTES
        achieved = bytes13 / (g13.value * 1e-3) / 1e9 if g13.value > 0 else None
        bytes2 = float(sum(steps_uniq)) * W2_BYTES
        achieved2 = bytes2 / (g2.value * 1e-3) / 1e9 if g2.value > 0 else None
        line = {
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": K,
            "warmup": Wm, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 accumulate over E2M1xE4M3 / E4M3xE4M3 tensor-core products",
            "data": "synthetic", "config": workload_config(a, world), "clocks": clocks,
            "e2e": {"value": e2e_val, "unit": "tok/s", "h2d_bytes_per_step": world * T * W.dim * 4,
                    "d2h_bytes_per_step": world * T * W.dim * 4},
            "gpu_launches": launches,
            "roofline": {"kernel": ("gemm_tc_kernel<pair> (tcgen05 block-scaled MXFP4 expert gate/up GEMV + SwiGLU)"
                                    if L.apus_cuda_moe_use_tc(handle, -1) == 1 else
                                    "gemm_small_kernel<MXFP4, pair> (mma.sync expert gate/up GEMV + SwiGLU)"),
                         "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": (achieved / peak) if achieved else None, "peak_kind": peak_kind,
                         "traffic": None, "launches": nl.value,
                         "avg_launch_us": g13.value / max(nl.value, 1) * 1e3,
                         "avg_unique_experts": float(np.mean(steps_uniq)),
                         "down_proj_kernel": {"achieved": achieved2, "frac": (achieved2 / peak) if achieved2 else None,
                                              "avg_launch_us": g2.value / max(nl.value, 1) * 1e3}},
        }
        if world == 1 and not a.no_cpu_baseline:
            os.environ.setdefault("APUS_THREADS", str(min(os.cpu_count() or 1, 32)))
            run, kind, cores = cpu_moe_runner(W, T)
            v, n, dt = time_cpu(run, T, budget_s=12.0, min_steps=2, max_steps=40)
            line["cpu_baseline"] = {"value": v, "unit": "tok/s", "cores": cores(), "kind": kind,
                                    "sample": f"{n} steps of T={T} tokens through apus_moe_forward on the host "
                                              f"cores in {dt:.1f} s"}
        emit(line)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
