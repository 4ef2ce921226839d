"""Consumer of the compiler's route-native MoE node chain.

The reference compiler lowers a sparse-expert feed-forward block into a list of circuit nodes
(nerve/circuit_lowering_sparse_experts.py:7-211):

    linear -> moe_route -> independent_sparse_moe_gate_up -> independent_sparse_moe_down -> moe_reduce
    (+ parameter_table_resource_preselection in front for token-id-table routing,
     + linear, linear, (bounded_)silu_multiply, linear, residual_add for the dense shared expert)

and its runtime validates that chain before it builds kernel steps from it
(runtime-rs/src/vulkan_stream_circuit/sparse_moe_execution.rs:9-145) and derives the router's template
constants from the node attributes (nerve/model_package_moe_routing.py:18-213).  This module does the
same three things for the CUDA backend: it validates the chain with the reference's rules and error
texts, turns the attributes into an ``nvmoe_geometry``, and lists, node by node, the C entry point
that replaces the node's kernel together with the signals and parameters it binds, in the reference's
binding order (runtime-rs/src/vulkan_stream_circuit/circuit_binding_builder.rs:1-96).  Host logic only:
nothing here touches a device.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass, field

from . import capi

ROUTER_SCORE_TOPK, ROUTER_TOPK_SOFTMAX, ROUTER_TOPK_ROUTED, ROUTER_PRESELECTED = 0, 1, 2, 3
ACTIVATIONS = {"sigmoid": 0, "softmax": 1, "sqrtsoftplus": 2}
BIAS_DTYPES = {None: 0, "F32": 1, "BF16": 2}


class ChainError(ValueError):
    """Counterpart of the reference's package errors (``VulkanResidentTokenModelPackageError``,
    ``ModelCompileError``): the message names the node and the rule it breaks."""


def _moe_error(node: dict, message: str) -> ChainError:
    return ChainError(f"sparse MoE node {node.get('id')!r} {message}")


def _attr_usize(node: dict, attr: str) -> int:
    value = node.get("attrs", {}).get(attr)
    if isinstance(value, bool) or not isinstance(value, int) or value < 0:
        raise ChainError(f"sparse MoE node {node.get('id')!r} has no valid {attr!r} attribute")
    return value


def sparse_moe_geometry(node: dict):
    """(declared experts, selected routes per token) of a gate/up node, None for any other node
    (sparse_moe_execution.rs:42-86)."""
    op = node.get("op")
    if op not in ("sparse_moe_gate_up", "independent_sparse_moe_gate_up"):
        return None
    selected = _attr_usize(node, "experts_per_token")
    if op == "sparse_moe_gate_up":
        return _attr_usize(node, "num_experts"), selected
    accesses = node.get("attrs", {}).get("selected_parameter_accesses")
    if not isinstance(accesses, list):
        raise _moe_error(node, "has no selected-parameter access")
    if len(accesses) != 1:
        raise _moe_error(node, "requires exactly one selected-parameter access")
    mapping = accesses[0].get("mapping")
    if not isinstance(mapping, list):
        raise _moe_error(node, "has no selected-resource mapping")
    if not mapping or any(entry.get("selector") != selector or not isinstance(entry.get("parameter_ids"), list)
                          or not entry["parameter_ids"] for selector, entry in enumerate(mapping)):
        raise _moe_error(node, "does not map every selected resource exactly once")
    return len(mapping), selected


def _require_one(nodes, gate_up, role, predicate):
    matching = [n for n in nodes if predicate(n)]
    if len(matching) != 1:
        raise _moe_error(gate_up, f"resolves {len(matching)} {role} nodes")
    return matching[0]


def validate_sparse_moe_execution_chain(nodes: list, gate_up: dict) -> dict:
    """The reference's chain rule (sparse_moe_execution.rs:89-145): the gate/up node names a routed
    execution signal among its inputs; exactly one router publishes it; exactly one down projection of the
    matching kind consumes the gate/up output and that signal; exactly one ``moe_reduce`` consumes the down
    output.  Returns {"router", "gate_up", "down", "reduce", "route_signal"}."""
    if gate_up.get("op") == "independent_sparse_moe_gate_up":
        accesses = gate_up.get("attrs", {}).get("selected_parameter_accesses") or [{}]
        route_signal = accesses[0].get("execution_signal")
    else:
        route_signal = (gate_up.get("inputs") or [None, None])[1] if len(gate_up.get("inputs", [])) > 1 else None
    if not isinstance(route_signal, str) or route_signal not in gate_up.get("inputs", []):
        raise _moe_error(gate_up, "has no routed execution signal")
    if len(gate_up.get("outputs", [])) != 1:
        raise _moe_error(gate_up, "must publish exactly one expert intermediate")
    gate_output = gate_up["outputs"][0]
    router = _require_one(nodes, gate_up, "router",
                          lambda n: n.get("op") in ("moe_route", "moe_topk") and route_signal in n.get("outputs", []))
    down_op = "independent_sparse_moe_down" if gate_up["op"] == "independent_sparse_moe_gate_up" else "sparse_moe_down"
    down = _require_one(nodes, gate_up, "down projection",
                        lambda n: n.get("op") == down_op and gate_output in n.get("inputs", [])
                        and route_signal in n.get("inputs", []))
    if len(down.get("outputs", [])) != 1:
        raise _moe_error(down, "must publish exactly one routed expert output")
    down_output = down["outputs"][0]
    reduce = _require_one(nodes, gate_up, "reduction",
                          lambda n: n.get("op") == "moe_reduce" and down_output in n.get("inputs", []))
    return {"router": router, "gate_up": gate_up, "down": down, "reduce": reduce, "route_signal": route_signal}


def routing_geometry(node: dict):
    """(routed resources, routed selections, always count, always weight, total resources, total selections)
    of a ``moe_route`` / preselection node, with the reference's checks (model_package_moe_routing.py:160-213)."""
    attrs = node.get("attrs", {})
    routed = int(attrs.get("routed_resource_count", 0))
    k = int(attrs.get("routed_selection_count", 0))
    always = attrs.get("always_selected_resources")
    if not 0 < k <= routed <= 4096 or not isinstance(always, list):
        raise ChainError(f"independent MoE routing node {node.get('id')!r} has invalid routing geometry r{routed} k{k}")
    weights = []
    for offset, resource in enumerate(always):
        weight = float(resource.get("weight", 0.0)) if isinstance(resource, dict) else 0.0
        if (not isinstance(resource, dict) or set(resource) != {"resource_index", "weight"}
                or resource.get("resource_index") != routed + offset or not math.isfinite(weight) or weight <= 0.0):
            raise ChainError(f"independent MoE routing node {node.get('id')!r} has a malformed always-selected "
                             f"resource at offset {offset}")
        weights.append(weight)
    if weights and len(set(weights)) != 1:
        raise ChainError(f"independent MoE routing node {node.get('id')!r} requires one common always-selected "
                         "resource weight")
    total_resources, total_selections = routed + len(always), k + len(always)
    if (total_resources > 4096 or int(attrs.get("experts_per_token", 0)) != total_selections
            or len(node.get("outputs", [])) != 1):
        raise ChainError(f"independent MoE routing node {node.get('id')!r} has inconsistent total geometry")
    return routed, k, len(always), weights[0] if weights else 1.0, total_resources, total_selections


def _validate_selection_domain(node: dict, total_resources: int, total_selections: int) -> None:
    expected = {
        "id": "experts", "resource_count": total_resources, "selection_signal": node["outputs"][0],
        "encoding": {"element_type": "u32", "selection_count_per_activation": total_selections, "index_shift": 0,
                     "index_mask": (1 << (total_resources - 1).bit_length()) - 1, "calibration_word_base": 0},
    }
    if node.get("attrs", {}).get("selection_domain") != expected:
        raise ChainError(f"independent MoE routing node {node.get('id')!r} has an inconsistent total "
                         "selection-domain contract")


@dataclass
class DispatchStep:
    """One call of the C ABI standing for one circuit node (or for a scheduler stage in front of it)."""

    node_id: str
    op: str
    entry: str                      # exported symbol of libnerve_cuda_moe.so
    bindings: list                  # [(binding name of the entry point, signal or parameter id or None)]
    note: str = ""
    scalars: dict = field(default_factory=dict)  # the entry point's scalar arguments, by name


@dataclass
class LayerDispatch:
    geometry: capi.Geometry
    steps: list = field(default_factory=list)
    signals: dict = field(default_factory=dict)        # role -> signal name
    gate_up_parameters: list = field(default_factory=list)  # [expert][w1, w1 scale, w3, w3 scale] parameter ids
    down_parameters: list = field(default_factory=list)     # [expert][w2, w2 scale]
    router_selection: str = ""
    shared_expert: bool = False
    preselection_table_rows: int = 0


def _router_fields(router: dict, bias_dtype):
    """router_kind, activation, normalize, scale, softcap, bias dtype, and the geometry counts of a router node."""
    attrs = router.get("attrs", {})
    if router["op"] == "moe_topk":
        # the packed-bank router form (nerve/circuit_lowering_nodes.py:611-640, model_package_shader_selection.py:1847-1892)
        activation = str(attrs.get("activation"))
        if activation not in ("sigmoid", "softmax"):
            raise ChainError(f"MoE router node {router.get('id')!r} has unsupported activation {activation!r}")
        softcap = float(attrs.get("logit_softcap", 0.0))
        if not math.isfinite(softcap) or softcap < 0.0:
            raise ChainError(f"MoE router node {router.get('id')!r} has invalid logit softcap {softcap}")
        has_bias = bool(attrs.get("selection_bias"))
        if has_bias and len(router.get("params", [])) != 1:
            raise ChainError(f"MoE router node {router.get('id')!r} is missing its selection bias")
        if not has_bias and router.get("params"):
            raise ChainError(f"MoE router node {router.get('id')!r} has an undeclared selection bias")
        normalize = bool(attrs.get("normalize_selected"))
        plain = activation == "softmax" and normalize and softcap == 0.0 and not has_bias
        kind = ROUTER_TOPK_SOFTMAX if plain else ROUTER_TOPK_ROUTED
        experts, k = _attr_usize(router, "num_experts"), _attr_usize(router, "experts_per_token")
        if not 0 < k <= experts <= 4096:
            raise ChainError(f"invalid sparse expert routing e{experts} k{k}")
        return dict(kind=kind, activation=ACTIVATIONS[activation], normalize=normalize, scale=1.0, softcap=softcap,
                    bias=BIAS_DTYPES[bias_dtype if has_bias else None], routed=experts, k=k, always=0, always_weight=1.0,
                    selection="topk")
    routed, k, always, always_weight, total_resources, total_selections = routing_geometry(router)
    selection = str(attrs.get("selection", ""))
    activation = str(attrs.get("activation", ""))
    scale = float(attrs.get("routed_scaling_factor", 0.0))
    if activation not in ACTIVATIONS:
        raise ChainError(f"independent MoE router node {router.get('id')!r} has unsupported activation {activation!r}")
    if not math.isfinite(scale) or scale <= 0.0:
        raise ChainError(f"independent MoE router node {router.get('id')!r} has invalid routed scale {scale}")
    if selection == "score_topk":
        _validate_selection_domain(router, total_resources, total_selections)
        if len(router.get("inputs", [])) != 1 or len(router.get("params", [])) != 1:
            raise ChainError(f"score-selected MoE router node {router.get('id')!r} requires router logits and one "
                             "selection-bias parameter")
        if bias_dtype not in ("F32", "BF16"):
            raise ChainError(f"score-selected MoE router node {router.get('id')!r} has an incompatible selection bias")
        kind, bias = ROUTER_SCORE_TOPK, BIAS_DTYPES[bias_dtype]
    elif selection == "preselected_resource_indices":
        if activation == "softmax":
            raise ChainError(f"preselected MoE router node {router.get('id')!r} requires an independently evaluable "
                             "activation")
        if len(router.get("inputs", [])) != 2 or router.get("params"):
            raise ChainError(f"preselected MoE router node {router.get('id')!r} requires router logits and exact "
                             "resource indices without parameters")
        kind, bias = ROUTER_PRESELECTED, 0
    else:
        raise ChainError(f"independent MoE router node {router.get('id')!r} has unsupported selection mode {selection!r}")
    return dict(kind=kind, activation=ACTIVATIONS[activation], normalize=bool(attrs.get("normalize_selected")), scale=scale,
                softcap=0.0, bias=bias, routed=routed, k=k, always=always, always_weight=always_weight, selection=selection)


def plan_from_nodes(nodes: list, *, max_tokens: int, selection_bias_dtype: str | None = "F32", act_block: int = 128,
                    preselection_table_rows: int = 0, preselection_table_word_stride: int = 1, swiglu_alpha: float = 1.0,
                    swiglu_up_offset: float = 0.0, n_group: int = 0, topk_group: int = 0) -> LayerDispatch:
    """Validates the node list of one route-native MoE body and returns its geometry and dispatch list.

    ``selection_bias_dtype`` is the packaged dtype of the router's selection-bias parameter ("F32",
    "BF16", or None) and ``preselection_table_rows`` / ``preselection_table_word_stride`` the shape and
    element width (1 = I32, 2 = I64) of a token-id routing table: the compiler reads these from the tensor
    index.  The remaining keyword arguments are the extensions of this backend that no node attribute
    carries (their defaults are the reference).
    """
    gate_ups = [n for n in nodes if sparse_moe_geometry(n) is not None]
    if len(gate_ups) != 1:
        raise ChainError(f"the node list holds {len(gate_ups)} sparse MoE gate/up nodes, one body has exactly one")
    gate_up = gate_ups[0]
    if gate_up["op"] != "independent_sparse_moe_gate_up":
        raise ChainError(f"sparse MoE node {gate_up.get('id')!r} uses packed expert banks, which this backend does not take: "
                         "experts must be independent resources (independent_sparse_moe_gate_up)")
    declared, selected = sparse_moe_geometry(gate_up)
    if selected == 0 or selected > declared:
        raise ChainError(f"sparse MoE node {gate_up.get('id')!r} selects {selected} routes from {declared} experts")
    chain = validate_sparse_moe_execution_chain(nodes, gate_up)
    router, down, reduce = chain["router"], chain["down"], chain["reduce"]
    r = _router_fields(router, selection_bias_dtype)

    # the sizes every node states must agree (the reference bakes each node's own copy into its shader)
    total_k = r["k"] + r["always"]
    total_resources = r["routed"] + r["always"]
    if total_resources != declared:
        raise _moe_error(gate_up, f"maps {declared} resources but its router publishes {total_resources}")
    for node in (gate_up, down, reduce):
        if _attr_usize(node, "experts_per_token") != total_k:
            raise _moe_error(node, f"states {node['attrs']['experts_per_token']} routes per token, its router selects {total_k}")
    if sparse_moe_down_mapping(down) != declared:
        raise _moe_error(down, "does not map the same resources as its gate/up node")
    hidden, intermediate = _attr_usize(gate_up, "hidden_size"), _attr_usize(gate_up, "intermediate_size")
    if (_attr_usize(down, "hidden_size"), _attr_usize(down, "intermediate_size")) != (hidden, intermediate):
        raise _moe_error(down, "disagrees with its gate/up node about the hidden or intermediate size")
    if _attr_usize(reduce, "hidden_size") != hidden:
        raise _moe_error(reduce, "disagrees with its gate/up node about the hidden size")
    reduce_scale = float(reduce["attrs"].get("routed_scaling_factor", 1.0))
    already = bool(reduce["attrs"].get("routing_weights_already_scaled"))
    if router["op"] == "moe_route" and not (already and reduce_scale == 1.0):
        # the router applied routed_scaling_factor to the weights (circuit_lowering_sparse_experts.py:166-171)
        raise _moe_error(reduce, "must not scale again: its router already applied the routed scaling factor")
    limit = float(gate_up["attrs"].get("swiglu_limit", 0.0))

    g = capi.Geometry()
    capi.load().nvmoe_geometry_default(ctypes.byref(g), hidden, intermediate, r["routed"], r["k"])
    g.always_count, g.always_weight = r["always"], r["always_weight"]
    g.router_kind, g.activation, g.normalize_selected = r["kind"], r["activation"], int(r["normalize"])
    g.bias_dtype, g.routed_scale, g.logit_softcap = r["bias"], r["scale"], r["softcap"]
    g.n_group, g.topk_group = n_group, topk_group
    g.swiglu_limit, g.swiglu_alpha, g.swiglu_up_offset = limit, swiglu_alpha, swiglu_up_offset
    g.act_block, g.reduce_scale, g.max_tokens = act_block, reduce_scale, max_tokens

    gate_mapping = gate_up["attrs"]["selected_parameter_accesses"][0]["mapping"]
    down_mapping = down["attrs"]["selected_parameter_accesses"][0]["mapping"]
    for node, mapping, per in ((gate_up, gate_mapping, 4), (down, down_mapping, 2)):
        if any(len(entry["parameter_ids"]) != per for entry in mapping):
            raise _moe_error(node, f"must bind {per} parameters per resource (MXFP4 codes and E8M0 scales of "
                                   f"{'w1 and w3' if per == 4 else 'w2'})")
    out = LayerDispatch(geometry=g, router_selection=r["selection"], preselection_table_rows=preselection_table_rows,
                        gate_up_parameters=[list(e["parameter_ids"]) for e in gate_mapping],
                        down_parameters=[list(e["parameter_ids"]) for e in down_mapping])
    hidden_signal = gate_up["inputs"][0]
    route_signal = chain["route_signal"]
    out.signals = {"hidden": hidden_signal, "routes": route_signal, "intermediates": gate_up["outputs"][0],
                   "expert_outputs": down["outputs"][0], "output": reduce["outputs"][0]}

    steps = out.steps
    logits_signal = router["inputs"][0]
    projection = [n for n in nodes if n.get("op") == "linear" and logits_signal in n.get("outputs", [])]
    if len(projection) == 1:
        p = projection[0]
        out.signals["logits"] = logits_signal
        steps.append(DispatchStep(p["id"], "linear", "nvmoe_router_linear",
                                  [("hidden", p["inputs"][0]), ("logits", logits_signal), ("router_weights", p["params"][0]),
                                   ("router_bias", next((x for x in p["params"][1:] if x.endswith("_bias")), None))]))
    if r["kind"] == ROUTER_PRESELECTED:
        pre_signal = router["inputs"][1]
        pre = [n for n in nodes if n.get("op") == "parameter_table_resource_preselection" and pre_signal in n.get("outputs", [])]
        if len(pre) != 1:
            raise _moe_error(router, f"resolves {len(pre)} resource preselection nodes")
        pre = pre[0]
        pr = routing_geometry(pre)
        _validate_selection_domain(pre, pr[4], pr[5])
        dependency = pre["attrs"].get("predictable_dependency")
        expected = {"schema": "nerve.predictable_resource_selection.v1", "kind": "parameter_table_lookup",
                    "key_signal": pre["inputs"][0] if len(pre.get("inputs", [])) == 1 else "",
                    "table_parameter": pre["params"][0] if len(pre.get("params", [])) == 1 else "",
                    "selection_semantics": "exact"}
        if len(pre.get("inputs", [])) != 1 or len(pre.get("params", [])) != 1 or dependency != expected:
            raise ChainError(f"resource preselection node {pre.get('id')!r} has an invalid predictable dependency contract")
        if pr[:3] != (r["routed"], r["k"], r["always"]):
            raise _moe_error(router, "disagrees with its preselection node about the routing geometry")
        out.signals["token_ids"], out.signals["resource_routes"] = pre["inputs"][0], pre_signal
        steps.insert(0, DispatchStep(pre["id"], pre["op"], "nvmoe_resource_preselect_table",
                                     [("token_ids", pre["inputs"][0]), ("resource_routes", pre_signal),
                                      ("table", pre["params"][0]), ("telemetry", None)],
                                     scalars={"vocab_size": preselection_table_rows, "table_word_stride": preselection_table_word_stride}))
        steps.append(DispatchStep(router["id"], router["op"], "nvmoe_route_preselected",
                                  [("logits", logits_signal), ("resource_routes", pre_signal), ("routes", route_signal),
                                   ("telemetry", None)]))
    else:
        steps.append(DispatchStep(router["id"], router["op"], "nvmoe_route",
                                  [("logits", logits_signal), ("routes", route_signal),
                                   ("bias", router["params"][0] if router.get("params") else None), ("telemetry", None)]))
    steps.append(DispatchStep(gate_up["id"], "moe_route_compact", "nvmoe_route_compact",
                              [("routes", route_signal), ("intermediates", gate_up["outputs"][0]),
                               ("slots", f"{gate_up['id']}.parameter_slots"), ("control", f"{gate_up['id']}.control")],
                              note="scheduler stage in front of gate/up (moe_route_compact_batch1)"))
    steps.append(DispatchStep(gate_up["id"], gate_up["op"], "nvmoe_gate_up",
                              [("hidden", hidden_signal), ("routes", route_signal), ("intermediates", gate_up["outputs"][0]),
                               ("addresses", f"{gate_up['id']}.address_table"), ("slots", f"{gate_up['id']}.parameter_slots"),
                               ("control", f"{gate_up['id']}.control")]))
    steps.append(DispatchStep(down["id"], "moe_route_count", "nvmoe_route_count",
                              [("routes", route_signal), ("slots", f"{down['id']}.parameter_slots"),
                               ("control", f"{down['id']}.control")],
                              note="scheduler stage in front of down (moe_route_count_batch1)"))
    steps.append(DispatchStep(down["id"], down["op"], "nvmoe_down",
                              [("intermediates", gate_up["outputs"][0]), ("routes", route_signal),
                               ("outputs", down["outputs"][0]), ("addresses", f"{down['id']}.address_table"),
                               ("slots", f"{down['id']}.parameter_slots"), ("control", f"{down['id']}.control")]))
    steps.append(DispatchStep(reduce["id"], reduce["op"], "nvmoe_reduce",
                              [("expert_outputs", down["outputs"][0]), ("output", reduce["outputs"][0])]))
    _shared_expert_steps(nodes, hidden_signal, reduce["outputs"][0], intermediate, limit, out)
    return out


def sparse_moe_down_mapping(down: dict) -> int:
    accesses = down.get("attrs", {}).get("selected_parameter_accesses")
    if not isinstance(accesses, list) or len(accesses) != 1 or not isinstance(accesses[0].get("mapping"), list):
        raise _moe_error(down, "requires exactly one selected-parameter access")
    mapping = accesses[0]["mapping"]
    if not mapping or any(entry.get("selector") != i or not entry.get("parameter_ids") for i, entry in enumerate(mapping)):
        raise _moe_error(down, "does not map every selected resource exactly once")
    return len(mapping)


def _shared_expert_steps(nodes, hidden_signal, routed_signal, intermediate, limit, out: LayerDispatch) -> None:
    """The dense shared expert beside the routed ones (circuit_lowering_sparse_experts.py:173-209): two
    projections of the normed hidden state, (bounded) SiLU-multiply, the down projection, and the add that
    joins it to the routed output."""
    add = [n for n in nodes if n.get("op") == "residual_add" and routed_signal in n.get("inputs", [])]
    if not add:
        return
    if len(add) != 1 or len(add[0]["inputs"]) != 2:
        raise ChainError(f"the routed output {routed_signal!r} feeds {len(add)} residual adds")
    add = add[0]
    shared_signal = next(s for s in add["inputs"] if s != routed_signal)

    def producer(signal, ops):
        found = [n for n in nodes if signal in n.get("outputs", []) and n.get("op") in ops]
        if len(found) != 1:
            raise ChainError(f"shared expert: signal {signal!r} has {len(found)} producers among {sorted(ops)}")
        return found[0]

    down = producer(shared_signal, {"linear"})
    act = producer(down["inputs"][0], {"silu_multiply", "bounded_silu_multiply"})
    gate, up = producer(act["inputs"][0], {"linear"}), producer(act["inputs"][1], {"linear"})
    if gate["inputs"][0] != hidden_signal or up["inputs"][0] != hidden_signal:
        raise ChainError("shared expert: the gate and up projections must read the signal the routed experts read")
    if int(act["attrs"].get("element_count", 0)) != intermediate:
        raise ChainError(f"shared expert activation {act.get('id')!r} covers {act['attrs'].get('element_count')} "
                         f"elements, the block's intermediate size is {intermediate}")
    act_limit = float(act["attrs"].get("limit", 0.0)) if act["op"] == "bounded_silu_multiply" else 0.0
    if act_limit != limit:
        raise ChainError(f"shared expert activation {act.get('id')!r} clamps at {act_limit}, the routed experts at {limit}")
    out.shared_expert = True
    out.signals.update({"shared_gate": gate["outputs"][0], "shared_up": up["outputs"][0], "shared_hidden": act["outputs"][0],
                        "shared_out": shared_signal, "ffn_out": add["outputs"][0]})
    hidden = out.geometry.hidden_size
    for node in (gate, up):
        out.steps.append(DispatchStep(node["id"], "linear", "nvmoe_dense_linear",
                                      [("input", node["inputs"][0]), ("output", node["outputs"][0]),
                                       ("weights", node["params"][0]), ("scales", node["params"][1] if len(node["params"]) > 1 else None)],
                                      scalars={"rows": intermediate, "cols": hidden}))
    out.steps.append(DispatchStep(act["id"], act["op"], "nvmoe_silu_multiply",
                                  [("gate", act["inputs"][0]), ("up", act["inputs"][1]), ("output", act["outputs"][0])],
                                  scalars={"element_count": intermediate, "limit": act_limit}))
    out.steps.append(DispatchStep(down["id"], "linear", "nvmoe_dense_linear",
                                  [("input", down["inputs"][0]), ("output", shared_signal), ("weights", down["params"][0]),
                                   ("scales", down["params"][1] if len(down["params"]) > 1 else None)],
                                  scalars={"rows": hidden, "cols": intermediate}))
    out.steps.append(DispatchStep(add["id"], "residual_add", "nvmoe_residual_add",
                                  [("a", add["inputs"][0]), ("b", add["inputs"][1]), ("output", add["outputs"][0])],
                                  scalars={"element_count": hidden}))
