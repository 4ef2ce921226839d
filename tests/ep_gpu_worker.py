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
        # split sizes read on the host / fixed segments over torch.distributed / the library's own collectives
        for mode in ("ragged", "padded", "native"):
            layer = ExpertParallelLayer(cfg, tokens, rank, world, local, seed=5, expert_path=path, mode=mode, dist=dist)
            for _ in range(2):  # the second step reuses every buffer
                sent, received = layer.step(dist)
            got = layer.output()
            same = np.array_equal(got, want)
            print(f"rank {rank} path {path} {mode}: sent {sent} received {received} parity {'ok' if same else 'FAILED'} "
                  f"({int((got != want).sum())} of {got.size} values differ)", flush=True)
            failures += 0 if same else 1
    flag = torch.tensor([failures], device=f"cuda:{local}")
    dist.all_reduce(flag)
    dist.destroy_process_group()
    return 1 if int(flag.item()) else 0


if __name__ == "__main__":
    sys.exit(main())
