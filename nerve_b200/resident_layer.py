"""One device's resident MoE layer: packaged expert tensors uploaded once, a plan, and the buffers of a
layer call.  What a runtime holds per mounted component (the reference's resident buffers plus resident
kernel dispatches, runtime-rs/src/vulkan_compute/resident_buffers.rs:39-232), packaged for the parity
tests and the benchmark, which both drive the layer through it.
"""
from __future__ import annotations

import time

import numpy as np

from . import synthetic
from .backend import CudaComputeDevice, ExpertBank, MoePlan

L2_BYTES = 126 * 1024 * 1024  # B200 L2


def upload_expert_banks(device, cfg, seed, owned, copies):
    """`copies` resident copies ("banks") of the experts in `owned`, generated and uploaded one expert at a
    time so that host memory stays flat however large the layer is."""
    banks = [[] for _ in range(copies)]
    n = cfg.total_experts
    for e in range(n):
        tensors = synthetic.expert_tensors(cfg, seed, e) if e in owned else None
        for bank in banks:
            bank.append(None if tensors is None else [device.resident_buffer_from(t) for t in tensors])
    return [ExpertBank.from_resident(device, per_expert) for per_expert in banks]


class LayerRunner:
    """One rank's resident layer: weights, plan, device buffers.

    Several resident copies of the layer's weights ("banks", as a model's successive layers would be) are
    visited in turn: the weights a step reads were last read a whole cycle ago, and the cycle is several
    times the L2 size, so every step streams its weights from HBM without dirtying L2 first.  A runner
    built with ``share=other`` reuses the other's device and banks (same config, another batch size).
    """

    def __init__(self, cfg, tokens, seed, expert_path, device_index=0, expert_start=0, expert_count=0, banks=0,
                 share: "LayerRunner | None" = None):
        self.cfg, self.tokens, self.seed = cfg, tokens, seed
        self.case = synthetic.make_case(cfg, tokens, seed=seed, with_weights=False)
        owned = range(cfg.total_experts) if not expert_count else range(expert_start, expert_start + expert_count)
        self.owned = list(owned)
        per_expert = cfg.expert_weight_bytes
        touched = max(1, min(tokens * cfg.total_k, len(self.owned))) * per_expert
        if share is not None:
            assert share.cfg.hidden == cfg.hidden and share.cfg.intermediate == cfg.intermediate and share.owned == self.owned
            self.device, self.banks = share.device, share.banks
        else:
            self.device = CudaComputeDevice(device_index)
            copies = banks or max(2, min(8, -(-4 * L2_BYTES // touched)))
            self.banks = upload_expert_banks(self.device, cfg, seed, set(self.owned), copies)
        self.n_banks = len(self.banks)
        self.bank = self.banks[0]
        self.cycle_bytes = touched * self.n_banks
        self.turn = 0
        self.plan = MoePlan.for_config(self.device, cfg, tokens)
        if expert_path:
            self.plan.set_expert_path(expert_path)
        self.plan.set_profiling(True)
        c = self.case
        self.hidden = self.device.resident_buffer_from(c.hidden)
        self.router_w = self.device.resident_buffer_from(c.router_w)
        self.router_bias = self.device.resident_buffer_from(c.router_bias) if c.router_bias is not None else None
        self.select_bias = self.device.resident_buffer_from(c.select_bias) if c.select_bias is not None else None
        self.output = self.device.create_resident_buffer(tokens * cfg.hidden * 2)
        self.routes = self.device.create_resident_buffer(tokens * cfg.total_k * 4)
        self.telemetry = self.device.create_resident_buffer(self.plan.telemetry_words() * 4)
        self.kw = dict(router_weights=self.router_w, router_bias=self.router_bias, bias=self.select_bias,
                       telemetry=self.telemetry, routes_out=self.routes, expert_start=expert_start,
                       expert_count=expert_count)
        self._pinned = None

    def _host_buffers(self):
        # the end-to-end call reads its tokens from, and writes its result to, page-locked host memory
        if self._pinned is None:
            import torch

            self._pinned = (torch.empty((self.tokens, self.cfg.hidden), dtype=torch.int16).pin_memory(),
                            torch.empty((self.tokens, self.cfg.hidden), dtype=torch.int16).pin_memory())
            self.hidden_host = self._pinned[0].numpy().view(np.uint16)
            self.hidden_host[...] = self.case.hidden
            self.out_host = self._pinned[1].numpy().view(np.uint16)
        return self.hidden_host, self.out_host

    def next_bank(self):
        self.turn += 1
        return self.banks[self.turn % self.n_banks]

    def step_resident(self) -> dict:
        self.plan.layer(self.tokens, self.next_bank(), self.hidden, self.output, **self.kw)
        return self.plan.last_report()

    def launch_step(self) -> None:
        """One layer call, nothing read back: the stream keeps running."""
        self.plan.layer(self.tokens, self.next_bank(), self.hidden, self.output, **self.kw)

    def step_host(self) -> float:
        hidden_host, out_host = self._host_buffers()
        bank = self.next_bank()
        t0 = time.perf_counter()
        self.plan.layer_host(self.tokens, bank, hidden_host, out_host, **self.kw)
        return (time.perf_counter() - t0) * 1e3

    def read_output(self) -> np.ndarray:
        return self.output.read(np.uint16).reshape(self.tokens, self.cfg.hidden)

    def read_routes(self) -> np.ndarray:
        return self.routes.read(np.uint32).reshape(self.tokens, self.cfg.total_k)

    def release(self) -> None:
        """Frees the plan and the per-call buffers (the banks and the device stay, for runners that share them)."""
        self.plan.destroy()
        for buf in (self.hidden, self.router_w, self.router_bias, self.select_bias, self.output, self.routes, self.telemetry):
            if buf is not None:
                buf.destroy()
