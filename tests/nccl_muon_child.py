"""One rank of the multi-GPU ``Muon.step`` tests (launched by torchrun): runs two steps and saves
the parameters; ``FM_MUON_GATHER`` selects the copy-engine or the NCCL all-gather."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests" / "golden"))
sys.path.insert(0, str(ROOT / "tests"))

from inputs import MUON_HP, MUON_SHAPES, muon_case  # noqa: E402
import flash_muon_b200 as fm  # noqa: E402


def main():
    rank, ws, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=ws)
    per = [(1024, 1024)] * 4 + [(4096, 1024), (1024, 4096)]
    steps = 2
    params, grads = muon_case(steps, shapes=MUON_SHAPES + per, seed=9)
    ps = [torch.nn.Parameter(p.cuda()) for p in params]
    opt = fm.Muon(ps, rank=rank, world_size=ws, **MUON_HP)
    for t in range(steps):
        for p, g in zip(ps, grads[t]):
            p.grad = g.cuda().clone()
        opt.step()
    torch.cuda.synchronize()
    fm._lib.device_status()
    dist.barrier()
    owned = sorted(i for i, p in enumerate(ps) if "momentum_buffer" in opt.state[p])
    mode = "peer" if opt._peer else "nccl"
    torch.save({"params": [p.detach().cpu() for p in ps], "owned": owned, "mode": mode},
               sys.argv[1] + f".rank{rank}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
