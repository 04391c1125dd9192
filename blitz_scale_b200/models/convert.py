"""Hugging Face Llama-family checkpoint (.safetensors) -> weight-segment files, one per TP rank.

    python -m blitz_scale_b200.models.convert --src /path/to/hf_model --model llama3_8b --out /data/llama3_8b --tp 2
    python -m blitz_scale_b200.models.convert --src /path/to/hf_model --list                      # tensor names, dtypes, shapes
    python -m blitz_scale_b200.models.convert --src ... --model ... --out ... --tp 2 --verify     # re-read and compare

What it does, like the reference's converter (scripts/util/make_dangertensors.py:9-30, 33-208): fixed tensor
order, every 2-D projection transposed to ``[in, out]``, gate and up fused, shards cut by head / intermediate
column / vocab row for every TP rank.  Differences: q, k and v are fused into one ``[hidden, (q + 2 kv) * hd]``
matrix, the output is the segment byte-for-byte (plus a JSON sidecar with the layout hash) and the source is read
through the native safetensors reader, which maps the files instead of loading them.

The rotary convention of Hugging Face Llama checkpoints (rotate-half) is the one the kernels use, so no permutation
of q/k rows is needed.
"""
from __future__ import annotations

import argparse
import json
import struct
import warnings
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from ..runtime import core
from .config import ModelConfig, get_config
from .weights import WeightSegment, shard_from_full

_DT = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64, "I64": torch.int64,
       "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
       "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2}
_ST = {v: k for k, v in _DT.items()}


class CheckpointReader:
    """All tensors of a directory of .safetensors shards (or of one file), by name."""

    def __init__(self, src):
        p = Path(src)
        files = sorted(p.glob("*.safetensors")) if p.is_dir() else [p]
        if not files:
            raise FileNotFoundError(f"no .safetensors under {src}")
        self.files = [core.SafeTensorsFile(str(f)) for f in files]
        self.where: Dict[str, int] = {}
        for i, f in enumerate(self.files):
            for n in f.names():
                self.where[n] = i

    def names(self) -> List[str]:
        return list(self.where)

    def __contains__(self, name: str) -> bool:
        return name in self.where

    def get(self, name: str) -> torch.Tensor:
        f = self.files[self.where[name]]
        info = f.info(name)
        view, _keep = f.view(name)
        if info.dtype not in _DT:
            raise TypeError(f"{name}: element type {info.dtype} is not supported")
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)      # the mapping is read-only; so are its users
            t = torch.frombuffer(view, dtype=_DT[info.dtype]) if info.nbytes else torch.empty(0, dtype=_DT[info.dtype])
        return t.reshape(tuple(info.shape))     # also right for 0-dimensional (scalar) tensors


def write_safetensors(path, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> None:
    """Minimal writer (tests, exporting a random-init model for other tools)."""
    header, off, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = metadata
    for name, t in tensors.items():
        t = t.contiguous().cpu()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _ST[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def hf_to_segment(reader: CheckpointReader, cfg: ModelConfig, dtype=torch.bfloat16) -> WeightSegment:
    """Full (tp=1) segment on the host from Hugging Face tensor names."""
    seg = WeightSegment(cfg, 1, 0, dtype, device="cpu")

    def w(name):  # [out, in] -> [in, out]
        return reader.get(name).to(dtype).t()

    seg["embed"].copy_(reader.get("model.embed_tokens.weight").to(dtype))
    for l in range(cfg.layers):
        s, d = f"model.layers.{l}.", f"layers.{l}."
        seg[d + "input_ln"].copy_(reader.get(s + "input_layernorm.weight").to(dtype))
        seg[d + "qkv"].copy_(torch.cat([w(s + "self_attn.q_proj.weight"), w(s + "self_attn.k_proj.weight"),
                                        w(s + "self_attn.v_proj.weight")], dim=1))
        seg[d + "o"].copy_(w(s + "self_attn.o_proj.weight"))
        seg[d + "post_ln"].copy_(reader.get(s + "post_attention_layernorm.weight").to(dtype))
        seg[d + "gate_up"].copy_(torch.cat([w(s + "mlp.gate_proj.weight"), w(s + "mlp.up_proj.weight")], dim=1))
        seg[d + "down"].copy_(w(s + "mlp.down_proj.weight"))
    seg["final_norm"].copy_(reader.get("model.norm.weight").to(dtype))
    head = "lm_head.weight" if "lm_head.weight" in reader else "model.embed_tokens.weight"  # tied embeddings
    seg["lm_head"].copy_(w(head))
    return seg


def segment_to_hf(seg: WeightSegment) -> Dict[str, torch.Tensor]:
    """Inverse mapping (export a segment under Hugging Face names)."""
    c = seg.cfg
    Q, K = c.q_heads * c.head_dim, c.kv_heads * c.head_dim
    out = {"model.embed_tokens.weight": seg["embed"].clone()}
    for l in range(c.layers):
        s, d = f"model.layers.{l}.", f"layers.{l}."
        qkv, gu = seg[d + "qkv"], seg[d + "gate_up"]
        out[s + "input_layernorm.weight"] = seg[d + "input_ln"].clone()
        out[s + "self_attn.q_proj.weight"] = qkv[:, :Q].t().contiguous()
        out[s + "self_attn.k_proj.weight"] = qkv[:, Q:Q + K].t().contiguous()
        out[s + "self_attn.v_proj.weight"] = qkv[:, Q + K:].t().contiguous()
        out[s + "self_attn.o_proj.weight"] = seg[d + "o"].t().contiguous()
        out[s + "post_attention_layernorm.weight"] = seg[d + "post_ln"].clone()
        out[s + "mlp.gate_proj.weight"] = gu[:, :c.inter].t().contiguous()
        out[s + "mlp.up_proj.weight"] = gu[:, c.inter:].t().contiguous()
        out[s + "mlp.down_proj.weight"] = seg[d + "down"].t().contiguous()
    out["model.norm.weight"] = seg["final_norm"].clone()
    out["lm_head.weight"] = seg["lm_head"].t().contiguous()
    return out


def convert(src, model: str, out_dir, tp: int = 1, dtype=torch.bfloat16) -> List[Path]:
    cfg = get_config(model)
    full = hf_to_segment(CheckpointReader(src), cfg, dtype)
    paths = []
    for r in range(tp):
        shard = full if tp == 1 else shard_from_full(full, tp, r, device="cpu")
        paths.append(shard.save(Path(out_dir) / (f"tp{tp}" if tp > 1 else "")))
    return paths


def list_checkpoint(src) -> List[Tuple[str, str, Tuple[int, ...]]]:
    """(name, dtype, shape) of every tensor of a checkpoint (the reference's read_safetensors helper)."""
    r = CheckpointReader(src)
    out = []
    for n in sorted(r.names()):
        info = r.files[r.where[n]].info(n)
        out.append((n, info.dtype, tuple(info.shape)))
    return out


def verify(src, model: str, out_dir, tp: int = 1, dtype=torch.bfloat16) -> List[str]:
    """Re-read the segment files under `out_dir` and compare every tensor of every TP rank with what the source
    checkpoint says it should be (the reference's check_dangertensors helper).  Returns the list of problems."""
    cfg = get_config(model)
    full = hf_to_segment(CheckpointReader(src), cfg, dtype)
    problems = []
    d = Path(out_dir) / (f"tp{tp}" if tp > 1 else "")
    for r in range(tp):
        want = full if tp == 1 else shard_from_full(full, tp, r, device="cpu")
        try:
            path = WeightSegment.check_sidecar(d, cfg, tp, r, dtype)
        except Exception as e:  # noqa: BLE001
            problems.append(f"rank {r}: {e}")
            continue
        got = WeightSegment(cfg, tp, r, dtype)
        n = got.layout.total_bytes
        if path.stat().st_size != n:
            problems.append(f"rank {r}: file has {path.stat().st_size} bytes, layout needs {n}")
            continue
        core.load_file_to_host(str(path), got.buffer.data_ptr(), n)
        for name in want.names():
            if not torch.equal(got[name], want[name]):
                diff = (got[name].float() - want[name].float()).abs().max().item()
                problems.append(f"rank {r}: {name} differs (max abs {diff:g})")
    return problems


def main(argv: Optional[Iterable[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--src", required=True, help="directory of .safetensors shards, or one file")
    ap.add_argument("--model", default="", help="registry name (llama3_8b, llama2_7b, mistral_24b, ...)")
    ap.add_argument("--out", default="")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--list", action="store_true", help="only list the tensors of the source checkpoint")
    ap.add_argument("--verify", action="store_true", help="do not write: compare the segment files under --out with the source")
    a = ap.parse_args(argv)
    if a.list:
        for n, dt, shape in list_checkpoint(a.src):
            print(f"{n}\t{dt}\t{list(shape)}")
        return 0
    if not a.model or not a.out:
        ap.error("--model and --out are required")
    dt = torch.bfloat16 if a.dtype == "bf16" else torch.float16
    if a.verify:
        problems = verify(a.src, a.model, a.out, a.tp, dt)
        for p in problems:
            print(p)
        print("ok" if not problems else f"{len(problems)} problem(s)")
        return 1 if problems else 0
    for p in convert(a.src, a.model, a.out, a.tp, dt):
        print(p)
    return 0


def cli(argv: Optional[Iterable[str]] = None) -> int:
    """`main` for the command line: what is wrong with the arguments or the files is one line, not a traceback."""
    try:
        return main(argv)
    except (OSError, KeyError, ValueError, RuntimeError) as e:   # missing source, unknown model, tensor of another shape
        raise SystemExit(f"convert: {e}")


if __name__ == "__main__":
    raise SystemExit(cli())
