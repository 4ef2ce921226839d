"""Seeded synthetic MoE layers with the shapes and value distributions of the benchmark configs.

No dataset, checkpoint or benchmark item is involved: shapes come from public model configs
(gpt-oss-20b/120b, DeepSeek-V3) and every tensor is drawn from ``numpy.random.Generator(PCG64)``
sub-streams named after the tensor, so that the checker, the CPU baseline and the CUDA path all
see identical bytes.

Value distributions
  activations  N(0,1) rounded to bf16 (round-to-nearest-even on the bit pattern)
  router W     N(0,0.02) bf16
  router bias  N(0,0.1) bf16, added inside the router projection (gpt-oss shapes)
  select bias  N(0,0.05) f32 (DeepSeek-V3 shape)
  MXFP4 codes  bytes uniform over 0..255 (both nibbles uniform over the 16 E2M1 values)
  E8M0 scales  bytes uniform over 121..127 (2^-6 .. 2^0)
  prefill skew expert popularity p_e ~ rank^-1.1 over a seeded permutation; log p_e is added to
               the router bias so that the realised top-k histogram is Zipf-skewed
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass, field, replace

import numpy as np

ROUTER_SCORE_TOPK, ROUTER_TOPK_SOFTMAX, ROUTER_TOPK_ROUTED = 0, 1, 2
ACT_SIGMOID, ACT_SOFTMAX, ACT_SQRT_SOFTPLUS = 0, 1, 2
BIAS_NONE, BIAS_F32, BIAS_BF16 = 0, 1, 2


@dataclass(frozen=True)
class MoeConfig:
    name: str
    hidden: int
    intermediate: int
    experts: int
    k: int
    router_kind: int = ROUTER_SCORE_TOPK
    activation: int = ACT_SOFTMAX
    normalize_selected: int = 1
    routed_scale: float = 1.0
    bias_dtype: int = BIAS_NONE        # selection bias handed to the router
    logit_bias: bool = False           # bf16 bias added by the router projection
    always_count: int = 0
    always_weight: float = 1.0
    n_group: int = 0
    topk_group: int = 0
    swiglu_limit: float = 0.0
    swiglu_alpha: float = 1.0
    swiglu_up_offset: float = 0.0
    act_block: int = 128
    zipf_s: float = 0.0
    logit_softcap: float = 0.0
    native_fp8_resources: int = 0      # resources at the end of the id range held as native FP8

    @property
    def total_k(self) -> int:
        return self.k + self.always_count

    @property
    def total_experts(self) -> int:
        return self.experts + self.always_count

    @property
    def expert_weight_bytes(self) -> int:
        """w1 + w3 + w2 codes and scales of one expert."""
        return 3 * self.hidden * self.intermediate * 17 // 32

    def reference_exact(self) -> "MoeConfig":
        """The same layer with every extension knob at its reference value."""
        return replace(self, n_group=0, topk_group=0, swiglu_alpha=1.0, swiglu_up_offset=0.0)


CONFIGS = {
    # BASELINE.json configs[0]
    "tiny": MoeConfig("tiny", 256, 512, 8, 2, ROUTER_SCORE_TOPK, ACT_SOFTMAX, 1, 1.0),
    # configs[1] and [2]: gpt-oss-20b shape, softmax over the selected k, logit bias, clamped SwiGLU
    "gpt-oss-20b": MoeConfig("gpt-oss-20b", 2880, 2880, 32, 4, ROUTER_TOPK_SOFTMAX, ACT_SOFTMAX, 1, 1.0,
                             logit_bias=True, swiglu_limit=7.0, swiglu_alpha=1.702,
                             swiglu_up_offset=1.0, act_block=32),
    "gpt-oss-20b-prefill": MoeConfig("gpt-oss-20b-prefill", 2880, 2880, 32, 4, ROUTER_TOPK_SOFTMAX,
                                     ACT_SOFTMAX, 1, 1.0, logit_bias=True, swiglu_limit=7.0,
                                     swiglu_alpha=1.702, swiglu_up_offset=1.0, act_block=32, zipf_s=1.1),
    # configs[3]
    "gpt-oss-120b": MoeConfig("gpt-oss-120b", 2880, 2880, 128, 4, ROUTER_TOPK_SOFTMAX, ACT_SOFTMAX, 1, 1.0,
                              logit_bias=True, swiglu_limit=7.0, swiglu_alpha=1.702,
                              swiglu_up_offset=1.0, act_block=32),
    # configs[4]
    "deepseek-v3": MoeConfig("deepseek-v3", 7168, 2048, 256, 8, ROUTER_SCORE_TOPK, ACT_SIGMOID, 1, 2.5,
                             bias_dtype=BIAS_F32, always_count=1, always_weight=1.0, n_group=8,
                             topk_group=4, act_block=128),
}


def small_variant(cfg: MoeConfig, hidden: int, intermediate: int, experts: int | None = None) -> MoeConfig:
    """The same routing and activation rules at sizes a CPU checks in seconds."""
    experts = cfg.experts if experts is None else experts
    n_group = cfg.n_group if cfg.n_group and experts % cfg.n_group == 0 else 0
    return replace(cfg, name=f"{cfg.name}-h{hidden}-i{intermediate}-e{experts}", hidden=hidden,
                   intermediate=intermediate, experts=experts, n_group=n_group,
                   topk_group=cfg.topk_group if n_group else 0)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (bits >> 16) & 1
    return (((bits + 0x7FFF + lsb) >> 16) & 0xFFFF).astype(np.uint16)


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _stream(seed: int, name: str) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64([seed, zlib.crc32(name.encode())]))


@dataclass
class MoeCase:
    cfg: MoeConfig
    tokens: int
    seed: int
    hidden: np.ndarray                 # [T,H] uint16 (bf16 bits)
    router_w: np.ndarray               # [E,H] uint16
    router_bias: np.ndarray | None     # [E] uint16, added by the projection
    select_bias: np.ndarray | None     # [E] float32 or uint16, handed to the router
    w1: list = field(default_factory=list)   # per expert [I,H/2] uint8
    s1: list = field(default_factory=list)   # per expert [I,H/32] uint8
    w3: list = field(default_factory=list)
    s3: list = field(default_factory=list)
    w2: list = field(default_factory=list)   # per expert [H,I/2] uint8
    s2: list = field(default_factory=list)   # per expert [H,I/32] uint8


def make_case(cfg: MoeConfig, tokens: int, seed: int = 0, with_weights: bool = True) -> MoeCase:
    H, I, E = cfg.hidden, cfg.intermediate, cfg.experts
    hidden = f32_to_bf16(_stream(seed, "hidden").standard_normal((tokens, H), dtype=np.float32))
    router_w = f32_to_bf16(0.02 * _stream(seed, "router_w").standard_normal((E, H), dtype=np.float32))
    router_bias = None
    if cfg.logit_bias or cfg.zipf_s > 0.0:
        bias = 0.1 * _stream(seed, "router_bias").standard_normal(E).astype(np.float32) if cfg.logit_bias \
            else np.zeros(E, dtype=np.float32)
        if cfg.zipf_s > 0.0:
            order = _stream(seed, "zipf_perm").permutation(E)
            p = np.empty(E, dtype=np.float64)
            p[order] = (np.arange(1, E + 1, dtype=np.float64)) ** (-cfg.zipf_s)
            p /= p.sum()
            bias = bias + np.log(p).astype(np.float32)
        router_bias = f32_to_bf16(bias)
    select_bias = None
    if cfg.bias_dtype == BIAS_F32:
        select_bias = (0.05 * _stream(seed, "select_bias").standard_normal(E)).astype(np.float32)
    elif cfg.bias_dtype == BIAS_BF16:
        select_bias = f32_to_bf16(0.05 * _stream(seed, "select_bias").standard_normal(E).astype(np.float32))
    case = MoeCase(cfg, tokens, seed, hidden, router_w, router_bias, select_bias)
    if with_weights:
        for e in range(cfg.total_experts):
            for name, tensor in zip(EXPERT_TENSOR_NAMES, expert_tensors(cfg, seed, e)):
                getattr(case, name).append(tensor)
    return case


EXPERT_TENSOR_NAMES = ("w1", "s1", "w3", "s3", "w2", "s2")


def expert_tensors(cfg: MoeConfig, seed: int, expert: int) -> tuple:
    """The six packaged tensors (w1, s1, w3, s3, w2, s2) of one expert, drawn from that expert's own
    sub-stream: any subset of the experts can be generated, in any order, and always holds the same bytes."""
    H, I = cfg.hidden, cfg.intermediate
    g = _stream(seed, f"expert{expert}")
    return (g.integers(0, 256, (I, H // 2), dtype=np.uint8), g.integers(121, 128, (I, H // 32), dtype=np.uint8),
            g.integers(0, 256, (I, H // 2), dtype=np.uint8), g.integers(121, 128, (I, H // 32), dtype=np.uint8),
            g.integers(0, 256, (H, I // 2), dtype=np.uint8), g.integers(121, 128, (H, I // 32), dtype=np.uint8))


E2M1_TO_E4M3 = np.array([0x00, 0x30, 0x38, 0x3C, 0x40, 0x44, 0x48, 0x4C, 0x80, 0xB0, 0xB8, 0xBC, 0xC0, 0xC4, 0xC8, 0xCC], dtype=np.uint8)


def expand_to_e4m3(packed: np.ndarray) -> np.ndarray:
    """The pre-expanded form of a packaged MXFP4 matrix: every E2M1 code as the E4M3 byte of the same value,
    low nibble first ([rows, cols/2] -> [rows, cols])."""
    out = np.empty((packed.shape[0], packed.shape[1] * 2), dtype=np.uint8)
    out[:, 0::2] = E2M1_TO_E4M3[packed & 0xF]
    out[:, 1::2] = E2M1_TO_E4M3[packed >> 4]
    return out


def native_fp8_tensors(cfg: MoeConfig, seed: int, expert: int) -> tuple:
    """A native FP8 resource: E4M3 weights [rows, cols] (finite codes only) with one E8M0 exponent byte per
    128 x 128 block, in the six-tensor order of `expert_tensors`."""
    H, I = cfg.hidden, cfg.intermediate
    g = _stream(seed, f"native_fp8_expert{expert}")

    def matrix(rows, cols):
        codes = g.integers(0, 256, (rows, cols), dtype=np.uint8)
        codes[(codes & 0x7F) == 0x7F] = 0x38  # S.1111.111 is NaN in E4M3
        scales = g.integers(112, 119, (-(-rows // 128), -(-cols // 128)), dtype=np.uint8)
        return codes, scales

    w1, s1 = matrix(I, H)
    w3, s3 = matrix(I, H)
    w2, s2 = matrix(H, I)
    return w1, s1, w3, s3, w2, s2


def expert_tensor_lists(cfg: MoeConfig, seed: int, experts, placeholder=None) -> dict:
    """name -> list over all resources, holding the tensors of `experts` and `placeholder` elsewhere."""
    w = {k: [placeholder] * cfg.total_experts for k in EXPERT_TENSOR_NAMES}
    for e in experts:
        for name, tensor in zip(EXPERT_TENSOR_NAMES, expert_tensors(cfg, seed, e)):
            w[name][e] = tensor
    return w


def expert_histogram(routes: np.ndarray, total_experts: int) -> np.ndarray:
    return np.bincount((routes.reshape(-1) & 0xFFFF).astype(np.int64), minlength=total_experts)
