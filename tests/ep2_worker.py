"""Worker of tests/test_gpu_ep2.py (one process per GPU, launched by torch.distributed.run):
the expert-parallel token loop over NCCL against the one-GPU loop on the same model.

Every rank holds its block of the routed experts of a three-layer model at the real
dimensions (256 experts per layer, hash and scored routing) and decodes its own
sequences; rank 0 then also builds the whole model on its GPU, decodes the job's
sequences there, and compares: the tokens must be the same, bit for bit, because the
exchange only moves rows and the combine adds in the reference's slot order."""
import ctypes as C
import datetime
import json
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def main():
    import torch
    import torch.distributed as dist
    import apus_b200
    from apus_b200 import capi
    from apus_b200.ep_model import EpModel
    from apus_b200.flash import FlashConfig, RandomFlashModel, prompt_ids
    out_path = sys.argv[1]
    world, rank, local = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    L = apus_b200.lib()
    err = C.create_string_buffer(512)
    assert L.apus_cuda_enable(err, 512) == 0, err.value
    cfg = FlashConfig()
    cfg.n_layers = 4                               # swa+hash, swa+hash, csa+hash, hca scored
    B, n_prompt, n_gen, max_pos = 3, 9, 20, 64
    per = cfg.n_experts // world
    W = RandomFlashModel(cfg, 0, dev, e_lo=rank * per, e_hi=(rank + 1) * per, max_pos=max_pos)
    ep = EpModel(W.desc, cfg.n_layers, cfg.n_experts, cfg.topk, cfg.dim, B, max_pos, rank, world, device=dev)
    ep.prefill(prompt_ids(0, rank * B, B, n_prompt, cfg.vocab))
    toks = torch.zeros(n_gen, B, dtype=torch.int64, device=dev)
    toks[0].copy_(ep.ids)
    for g in range(1, n_gen):
        if g == 4:
            ep.capture()                           # the rest of the steps replay one CUDA graph (NCCL inside)
        ep.step()
        toks[g].copy_(ep.ids)
    torch.cuda.synchronize()
    mine = toks.t().contiguous()
    gathered = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    ep.graph = None
    ep.close()
    dist.barrier()
    result = {"world": world}
    if rank == 0:
        got = torch.cat(gathered).cpu().numpy()                         # [world * B, n_gen]
        del W
        torch.cuda.empty_cache()
        Wf = RandomFlashModel(cfg, 0, dev, max_pos=max_pos)
        h = L.apus_cuda_model_create(C.byref(Wf.desc), world * B, max_pos)
        assert h, L.apus_cuda_last_error()
        want = np.zeros((world * B, n_gen), np.int32)
        ids = np.ascontiguousarray(prompt_ids(0, 0, world * B, n_prompt, cfg.vocab))
        assert L.apus_cuda_model_generate(h, capi.ptr(ids), n_prompt, n_gen, capi.ptr(want), None, None) == 0, \
            L.apus_cuda_last_error()
        L.apus_cuda_model_destroy(h)
        result.update(equal=bool(np.array_equal(got, want)), first_row_ep=got[0].tolist(), first_row_one=want[0].tolist(),
                      mismatches=int((got != want).sum()))
        Path(out_path).write_text(json.dumps(result))
    dist.barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
