"""Model shape registry and the per-rank weight-segment layout.

The registry mirrors the shapes the reference serves (src/model/common_hyper.h:11-177:
OPT, Llama-2 7B/13B/70B, Llama-3 8B, Mistral 13B/24B, Qwen 72B) plus the tiny shapes used by
the CPU plumbing configuration and the GPU unit tests.  Only the Llama architecture (pre-RMSNorm,
RoPE, GQA, SwiGLU, no biases) is executed, as in the reference, where every served model goes
through the Llama hyper-parameter constructor.

Weight segment (one contiguous allocation per GPU = per TP rank, every matrix stored ``[in, out]``
row-major, cf. src/model/llama.h:139-218 and scripts/util/make_dangertensors.py:9-30)::

    embed_tokens [vocab/tp, hidden]
    L x { input_ln [hidden] | qkv^T [hidden, (qh + 2 kvh)/tp * hd] | o^T [qh/tp * hd, hidden]
          | post_ln [hidden] | gate_up^T [hidden, 2 inter/tp] | down^T [inter/tp, hidden] }
    final_norm [hidden] | lm_head^T [hidden, vocab/tp]

Transfer units are ``embed | layer 0..L-1 | head`` (src/model/llama.h:236-246).  Two deliberate
differences from the reference layout: q, k and v projections are stored as one fused matrix whose
rows are ``[q | k | v]`` (one GEMM instead of two), and every tensor starts on a 256-byte boundary
(TMA operands need 16-byte alignment; 256 keeps copies sector-aligned).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Tuple

ALIGN_BYTES = 256


@dataclass(frozen=True)
class ModelConfig:
    name: str
    vocab: int
    hidden: int
    layers: int
    q_heads: int
    kv_heads: int
    head_dim: int
    inter: int
    rope_theta: float = 10000.0
    rms_eps: float = 1e-5
    max_positions: int = 16384
    param_gb: float = 0.0  # size used for flow accounting by the router
    eos_token: int = -1    # end-of-sequence id of the family's tokenizer (-1: none known); workers stop a request there
                           # unless it sets ignore_eos_token

    def kv_bytes_per_token(self, tp: int = 1, elem: int = 2) -> int:
        return 2 * (self.kv_heads // tp) * self.head_dim * elem * self.layers


# end-of-sequence ids of the published tokenizers: </s> = 2 (Llama-2, Mistral, OPT), <|end_of_text|> = 128001 (Llama-3),
# <|endoftext|> = 151643 (Qwen-2.5); a chat-tuned checkpoint that ends turns with another id sets --eos-token-id
_EOS = {"llama2": 2, "llama3": 128001, "mistral": 2, "qwen": 151643, "opt": 2, "tiny": 2}


def _c(name, vocab, hidden, layers, qh, kvh, inter, theta=10000.0, hd=None, gb=0.0, eps=1e-5):
    return ModelConfig(name, vocab, hidden, layers, qh, kvh, hd or hidden // qh, inter, theta, eps, 16384, gb,
                       _EOS.get(name.split("_")[0], -1))


REGISTRY: Dict[str, ModelConfig] = {c.name: c for c in [
    # CPU plumbing shape of the first benchmark configuration (2 layers, hidden 256, 4/2 heads, FFN 688)
    _c("tiny", 32000, 256, 2, 4, 2, 688),
    # smallest shape the tcgen05 attention (head_dim 128) accepts; used by GPU tests and smoke()
    _c("tiny_gpu", 4096, 512, 2, 4, 2, 1408, theta=5e5),
    _c("tiny_gpu_deep", 4096, 512, 8, 4, 2, 1408, theta=5e5),
    _c("tiny_gpu_wide", 4096, 1024, 2, 8, 4, 2816, theta=5e5),
    _c("opt_125m", 50272, 768, 12, 12, 12, 3072),
    _c("opt_1.3b", 50272, 2048, 24, 32, 32, 8192),
    _c("opt_6.7b", 50272, 4096, 32, 32, 32, 16384),
    _c("opt_13b", 50272, 5120, 40, 40, 40, 20480),
    _c("opt_30b", 50272, 7168, 48, 56, 56, 28672),
    _c("llama2_7b", 32000, 4096, 32, 32, 32, 11008, gb=14),
    _c("llama2_13b", 32000, 5120, 40, 40, 40, 13824, gb=26),
    _c("llama2_70b", 32000, 8192, 80, 64, 8, 28672, gb=140),
    _c("llama3_8b", 128256, 4096, 32, 32, 8, 14336, theta=5e5, gb=16),
    _c("mistral_13b", 32000, 5120, 40, 40, 8, 14336, theta=1e6, gb=26),
    _c("mistral_24b", 131072, 5120, 40, 32, 8, 32768, theta=1e8, hd=128, gb=48),
    _c("qwen_72b", 152064, 8192, 80, 64, 8, 29568, theta=1e6, gb=145, eps=1e-6),
]}


def get_config(name: str) -> ModelConfig:
    try:
        return REGISTRY[name]
    except KeyError:
        raise KeyError(f"unknown model {name!r}; known: {sorted(REGISTRY)}") from None


@dataclass
class TensorSpec:
    name: str
    shape: Tuple[int, ...]
    offset: int  # bytes from the start of the segment
    nbytes: int


@dataclass
class SegmentLayout:
    """Byte offsets of every tensor and of the transfer units of one TP rank's segment."""
    cfg: ModelConfig
    tp: int
    elem_bytes: int
    tensors: Dict[str, TensorSpec] = field(default_factory=dict)
    units: List[Tuple[str, int, int]] = field(default_factory=list)  # (name, offset, nbytes)
    total_bytes: int = 0

    def unit(self, name: str) -> Tuple[int, int]:
        for n, off, nb in self.units:
            if n == name:
                return off, nb
        raise KeyError(name)


def _align(x: int, a: int = ALIGN_BYTES) -> int:
    return (x + a - 1) // a * a


def layer_tensor_shapes(cfg: ModelConfig, tp: int) -> List[Tuple[str, Tuple[int, ...]]]:
    qh, kvh, hd = cfg.q_heads // tp, cfg.kv_heads // tp, cfg.head_dim
    return [
        ("input_ln", (cfg.hidden,)),
        ("qkv", (cfg.hidden, (qh + 2 * kvh) * hd)),
        ("o", (qh * hd, cfg.hidden)),
        ("post_ln", (cfg.hidden,)),
        ("gate_up", (cfg.hidden, 2 * (cfg.inter // tp))),
        ("down", (cfg.inter // tp, cfg.hidden)),
    ]


def build_layout(cfg: ModelConfig, tp: int = 1, elem_bytes: int = 2) -> SegmentLayout:
    if cfg.q_heads % tp or cfg.kv_heads % tp or cfg.inter % tp or cfg.vocab % tp:
        raise ValueError(f"{cfg.name}: heads/inter/vocab not divisible by tp={tp}")
    lay = SegmentLayout(cfg, tp, elem_bytes)
    cur = 0

    def add(name, shape):
        nonlocal cur
        n = 1
        for s in shape:
            n *= s
        nb = n * elem_bytes
        lay.tensors[name] = TensorSpec(name, tuple(shape), cur, nb)
        cur = _align(cur + nb)

    start = cur
    add("embed", (cfg.vocab // tp, cfg.hidden))
    lay.units.append(("embed", start, cur - start))
    for l in range(cfg.layers):
        start = cur
        for n, shp in layer_tensor_shapes(cfg, tp):
            add(f"layers.{l}.{n}", shp)
        lay.units.append((f"layer.{l}", start, cur - start))
    start = cur
    add("final_norm", (cfg.hidden,))
    add("lm_head", (cfg.hidden, cfg.vocab // tp))
    lay.units.append(("head", start, cur - start))
    lay.total_bytes = cur
    return lay
