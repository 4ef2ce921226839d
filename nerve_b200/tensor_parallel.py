"""Intra-expert tensor parallelism: every participant holds a range of the intermediate dimension of every
expert (the reference's ``tensor_parallel_expert`` strategy, nerve/model_package_physical_experts.py:98-327).

    replicated hidden + routes -> gate/up on the participant's rows of w1/w3 (its slice of the intermediates)
      -> down over the participant's columns of w2: raw f32 partial sums [T][K][H]
      -> the participants' planes gathered in participant order
      -> distributed_sum_f32_scale_packed_bf16: sum, scale by the route weight, one bf16 rounding
      -> moe_reduce

Ranges are aligned to 128 (INDEPENDENT_MXFP4_TP_COLUMNS), so the activation quantisation blocks of the down
stage are the unpartitioned ones and the result differs from one device only in the order of the f32 sum.
A participant is a plan whose intermediate_size is its range, over weight tensors that are its slices.
"""
from __future__ import annotations

from dataclasses import replace

import numpy as np

TP_ALIGNMENT = 128


def intermediate_ranges(intermediate: int, participants: int) -> list[tuple[int, int]]:
    """(start, count) of every participant: equal ranges, each a multiple of 128 columns."""
    if intermediate % (participants * TP_ALIGNMENT):
        raise ValueError(f"an intermediate size of {intermediate} does not split into {participants} ranges of whole "
                         f"{TP_ALIGNMENT}-column blocks")
    count = intermediate // participants
    return [(p * count, count) for p in range(participants)]


def slice_expert_tensors(tensors: tuple, start: int, count: int) -> tuple:
    """The participant's share of one expert's six packaged tensors: rows [start, start + count) of w1/w3 and
    their scales, columns [start, start + count) of w2 and its scales, each as a contiguous matrix of its own."""
    w1, s1, w3, s3, w2, s2 = tensors
    rows = slice(start, start + count)
    return (np.ascontiguousarray(w1[rows]), np.ascontiguousarray(s1[rows]), np.ascontiguousarray(w3[rows]),
            np.ascontiguousarray(s3[rows]), np.ascontiguousarray(w2[:, start // 2:(start + count) // 2]),
            np.ascontiguousarray(s2[:, start // 32:(start + count) // 32]))


class TensorParallelParticipant:
    """One participant's plan, weights and buffers on one device."""

    def __init__(self, device, cfg, max_tokens: int, participant: int, participants: int, expert_tensors, expert_path: int = 0):
        from .backend import ExpertBank, MoePlan

        self.device, self.cfg, self.participant, self.participants = device, cfg, participant, participants
        start, count = intermediate_ranges(cfg.intermediate, participants)[participant]
        self.local_cfg = replace(cfg, name=f"{cfg.name}-tp{participant}of{participants}", intermediate=count)
        self.plan = MoePlan.for_config(device, self.local_cfg, max_tokens)
        if expert_path:
            self.plan.set_expert_path(expert_path)
        per_expert = [[device.resident_buffer_from(t) for t in slice_expert_tensors(expert_tensors(e), start, count)]
                      for e in range(cfg.total_experts)]
        self.bank = ExpertBank.from_resident(device, per_expert)
        self.frames = device.create_resident_buffer(max_tokens * self.plan.frame_words * 4)
        self.gate_control = device.create_resident_buffer(28)
        self.down_control = device.create_resident_buffer(28)

    def partial_outputs(self, tokens: int, hidden, routes, partial_plane) -> None:
        """gate/up and the partial down projection of this participant into `partial_plane` [T][K][H] f32."""
        control = np.array([tokens, 0, 0, 0, 0, 0, 0], dtype=np.uint32)
        self.gate_control.write_bytes(control)
        self.down_control.write_bytes(control)
        p, b = self.plan, self.bank
        p.moe_route_compact(tokens, routes, self.frames, self.gate_control, b.gate_up_slots)
        p.independent_sparse_moe_gate_up(tokens, hidden, routes, self.frames, b.gate_up_addresses, b.gate_up_slots, self.gate_control)
        p.moe_route_count(tokens, routes, self.down_control, b.down_slots)
        p.independent_sparse_moe_down_partial(tokens, self.frames, routes, partial_plane, b.down_addresses, b.down_slots,
                                              self.down_control)


def finalize(plan, tokens: int, partial_planes, routes, expert_outputs, output, participants: int) -> None:
    """Sum of the participants' planes scaled by the route weights, then the combine, on the plan of the
    whole layer (any participant can do it: the planes and the routes are all it needs)."""
    K, H = plan.experts_per_token, plan.geometry.hidden_size
    plan.sum_f32_scale_packed_bf16(partial_planes, routes, expert_outputs, K * H, participants, tokens, H, 16)
    plan.moe_reduce(tokens, expert_outputs, output)
