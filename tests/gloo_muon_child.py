"""One CPU rank of ``test_muon_step_control_flow_over_gloo``.  ``Muon.step`` is the product's; the
four device hooks are replaced by the oracle's torch ops so the loop can run without a GPU."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests" / "golden"))

from inputs import MUON_HP, muon_case  # noqa: E402
from oracle import muon_oracle as O  # noqa: E402
import flash_muon_b200 as fm  # noqa: E402


class CpuMuon(fm.Muon):
    _buffer_device = "cpu"
    _rounds_per_pass = int(os.environ.get("TEST_ROUNDS_PER_PASS", "0"))

    def _momentum(self, g, buf, momentum, nesterov):
        return O.momentum_update(g, buf, momentum, nesterov)

    def _orthogonalize(self, g, out, steps):
        out.copy_(O.newtonschulz(g, steps=steps).flatten())

    def _all_gather(self, buffer, slot):
        # gloo wants a flat output and a non-aliasing input
        return dist.all_gather_into_tensor(buffer.view(-1), slot.clone(), async_op=True)

    def _apply_updates(self, params_world, views, lr, weight_decay):
        for p, g in zip(params_world, views):
            O.apply_update(p, g, lr, weight_decay)


def main():
    rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if ws > 1:
        dist.init_process_group("gloo", rank=rank, world_size=ws)
    steps = 2
    params, grads = muon_case(steps)
    opt = CpuMuon(params, rank=rank, world_size=ws, **MUON_HP)
    for t in range(steps):
        for p, g in zip(params, grads[t]):
            p.grad = g.clone()
        opt.step()
    owned = sorted(i for i, p in enumerate(params) if "momentum_buffer" in opt.state[p])
    torch.save({"params": [p.detach() for p in params], "owned": owned}, sys.argv[1] + f".rank{rank}")
    if ws > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
