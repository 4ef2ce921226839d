"""One rank of the multi-GPU expert-parallel parity check (launched by test_gpu_expert_parallel.py
through torch.distributed.run). Each rank computes its tokens with the experts sharded over the
ranks, then computes the whole batch alone with every expert resident on its own GPU, and demands
that its slice of the two results is bit-identical. Exit code 0 = parity."""
import os
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main() -> int:
    import torch
    import torch.distributed as dist

    from nerve_b200 import synthetic
    from nerve_b200.resident_layer import LayerRunner
    from nerve_b200.expert_parallel import ExpertParallelLayer

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    tokens = int(os.environ.get("NVMOE_EP_TOKENS", "24"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = synthetic.MoeConfig(name="ep-parity", hidden=512, intermediate=384, experts=8, k=2, act_block=32,
                              swiglu_limit=7.0, swiglu_alpha=1.702, swiglu_up_offset=1.0)
    failures = 0
    for path in (1, 2):
        alone = LayerRunner(cfg, tokens * world, 5, path, device_index=local, banks=1)
        alone.plan.layer(tokens * world, alone.bank, alone.hidden, alone.output, **alone.kw)
        want = alone.output.read(np.uint16).reshape(tokens * world, cfg.hidden)[rank * tokens:(rank + 1) * tokens]
        # split sizes read on the host / fixed segments over torch.distributed / the library's own collectives, the
        # last two also with segments bounded at 1.5 times the mean rows per peer
        for mode, factor in (("ragged", 0.0), ("padded", 0.0), ("native", 0.0), ("padded", 1.5), ("native", 1.5)):
            layer = ExpertParallelLayer(cfg, tokens, rank, world, local, seed=5, expert_path=path, mode=mode, dist=dist,
                                        capacity_factor=factor)
            for _ in range(2):  # the second step reuses every buffer
                sent, received = layer.step(dist)
            got = layer.output()
            same = np.array_equal(got, want) and not layer.overflowed()
            print(f"rank {rank} path {path} {mode} x{factor}: sent {sent} received {received} segment {layer.segment} "
                  f"parity {'ok' if same else 'FAILED'} ({int((got != want).sum())} of {got.size} values differ)", flush=True)
            failures += 0 if same else 1
        # segments far too small: the step completes, leaves the excess routes out and says so
        layer = ExpertParallelLayer(cfg, tokens, rank, world, local, seed=5, expert_path=path, mode="native", dist=dist,
                                    capacity_factor=0.25)
        layer.step(dist)
        layer.output()
        noticed = layer.overflowed()
        print(f"rank {rank} path {path} native x0.25: segment {layer.segment} overflow {'noticed' if noticed else 'MISSED'}", flush=True)
        failures += 0 if noticed else 1
    flag = torch.tensor([failures], device=f"cuda:{local}")
    dist.all_reduce(flag)
    dist.destroy_process_group()
    return 1 if int(flag.item()) else 0


if __name__ == "__main__":
    sys.exit(main())
