"""Worker of the expert-parallel tests (launched by torch.distributed.run, one process per GPU):
opens this rank's shard of a seeded synthetic model, decodes greedily and writes what it produced
to <out>/rank<r>.json.  Usage: ep_worker.py <out-dir> <cfg-json> <seed> <n-steps> [stall]

With "stall" the last rank stops issuing steps after the prompt (it stays alive and keeps its memory
mapped); the other ranks issue one more step, whose bounded wait for the stalled rank's row sums
runs out: the call must report BRRR_ERR_STATE (no hang, no fault) and the CUDA context must stay
usable.  Every rank closes its model only after a host barrier."""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    out_dir, cfg_json, seed, nsteps = sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4])
    stall = len(sys.argv) > 5 and sys.argv[5] == "stall"
    import torch
    import torch.distributed as dist
    import cpubrrr_b200 as B
    from cpubrrr_b200 import ep, synth as S
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = B.make_cfg(**json.loads(cfg_json))
    eng = ep.open_synth_ep(cfg, seed, rank, world, device=local, dist=dist, torch_device=dev)
    prompt = S.synth_prompt(seed, 9, cfg.n_vocab)
    first = eng.prefill(prompt)                                  # host-driven steps
    if stall:
        import time
        res = dict(first=int(first))
        if rank != world - 1:
            t0 = time.time()
            try:
                eng.run(first, len(prompt), True)
                res["error"] = None
            except B.BrrrError as e:
                res["error"] = str(e)
            res["seconds"] = time.time() - t0
            # the context is still usable: a fresh single-GPU model runs on the same device
            small = B.Engine.synth(B.make_cfg(128, 1, 4, 2, 8, 4, 512), 3, device=local)
            res["small_ok"] = int(small.run(1, 0, True)) < 512
            small.close()
        json.dump(res, open(os.path.join(out_dir, f"rank{rank}.json"), "w"))
        dist.barrier()                                           # nobody frees memory its peers may still write to
        eng.close()
        dist.destroy_process_group()
        return
    toks = [int(t) for t in eng.decode(first, len(prompt), nsteps)]   # device-chained steps
    res = dict(first=int(first), tokens=toks, hidden_bits=[int(b) for b in eng.hidden().view(np.uint32)],
               logit_bits=[int(b) for b in eng.logits().view(np.uint32)[:64]])
    json.dump(res, open(os.path.join(out_dir, f"rank{rank}.json"), "w"))
    dist.barrier()
    eng.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
