"""Low-precision checkpoints in and out, one tensor at a time:

    python -m halo_b200.checkpoint.tools.lowp_convert dequant-block-fp8 <src> <dst>
    python -m halo_b200.checkpoint.tools.lowp_convert export-block-fp8 <src> <dst> [--keep REGEX ...]
    python -m halo_b200.checkpoint.tools.lowp_convert export <src> <dst> --format mxfp8|mxfp4|nvfp4 [--keep REGEX ...]
    python -m halo_b200.checkpoint.tools.lowp_convert dequant <src> <dst>
    python -m halo_b200.checkpoint.tools.lowp_convert dequant-static-fp8 <src> <dst>
    python -m halo_b200.checkpoint.tools.lowp_convert dequant-mxfp4-experts <src> <dst>

``dequant-static-fp8`` reads releases with one static scale per matrix (or per expert of a bank);
``dequant-mxfp4-experts`` unpacks expert banks stored as ``<bank>_blocks`` / ``<bank>_scales`` (packed e2m1 codes with
one power-of-two scale per 32 values, the gpt-oss hub layout) into the bf16 banks the family's loader reads.
``dequant-block-fp8`` turns a served-weights release in 128 x 128 block FP8 (every ``<name>.weight`` in
``float8_e4m3fn`` beside a ``<name>.weight_scale_inv`` of one fp32 factor per block) into bf16 - the form training
starts from. ``export`` writes the matrices of a bf16 checkpoint in a block-scaled format: ``<name>.weight`` holds the
element codes, ``<name>.weight_scale`` the per-block scales and, for nvfp4, ``<name>.weight_global_scale`` the tensor
scale; embeddings, norms, router gates, biases and whatever ``--keep`` matches stay as they are. ``dequant`` reads
that layout back into bf16. The roles of the reference's fp8 / fp4 dequantisers and its low-precision exporters
(halo/checkpoint/tools/)."""

from __future__ import annotations

import argparse
import json
import os
import re
import sys

import torch

from halo_b200.ops import lowp

from ._io import CheckpointIndex, StreamingShardWriter, copy_side_files

BLOCK = 128
ALWAYS_KEPT = re.compile(r"(embed_tokens|lm_head|norm|\.gate\.weight$|shared_expert_gate|bias$|_hc\.|hc_head)")


def dequant_block_fp8(src: str, dst: str) -> int:
    idx = CheckpointIndex(src)
    writer = StreamingShardWriter(dst)
    n = 0
    for name in sorted(idx.weight_map):
        if name.endswith("_scale_inv"):
            continue
        t = idx.get(name)
        scale_name = name + "_scale_inv"
        if t.dtype == torch.float8_e4m3fn:
            if scale_name not in idx:
                raise KeyError(f"{name} is FP8 but {scale_name} is absent")
            s = idx.get(scale_name).float()
            rows, cols = t.shape
            if tuple(s.shape) != (-(-rows // BLOCK), -(-cols // BLOCK)):
                raise ValueError(f"{scale_name} is {tuple(s.shape)}, expected one factor per {BLOCK} x {BLOCK} block of {tuple(t.shape)}")
            full = s.repeat_interleave(BLOCK, 0)[:rows].repeat_interleave(BLOCK, 1)[:, :cols]
            t = (t.float() * full).to(torch.bfloat16)
            n += 1
        writer.add(name, t)
    writer.finish()
    copy_side_files(src, dst)
    cfg_path = os.path.join(dst, "config.json")
    if os.path.isfile(cfg_path):                               # the result is an ordinary bf16 checkpoint
        cfg = json.load(open(cfg_path))
        cfg.pop("quantization_config", None)
        cfg["torch_dtype"] = "bfloat16"
        json.dump(cfg, open(cfg_path, "w"), indent=2)
    return n


def _as_plain_bf16_config(dst: str) -> None:
    cfg_path = os.path.join(dst, "config.json")
    if os.path.isfile(cfg_path):
        cfg = json.load(open(cfg_path))
        cfg.pop("quantization_config", None)
        cfg["torch_dtype"] = "bfloat16"
        json.dump(cfg, open(cfg_path, "w"), indent=2)


def _reject_in_place(src: str, dst: str) -> None:
    if os.path.realpath(src) == os.path.realpath(dst):
        raise ValueError("the output directory is the input: the writer would delete the shards it is reading")


def dequant_static_fp8(src: str, dst: str) -> int:
    """Releases with STATIC scales: every ``<name>.weight`` in ``float8_e4m3fn`` beside a ``<name>.weight_scale`` that is
    one factor for the matrix, or one per expert for a 3-D bank ``[E, ...]``. ``weight = fp8 * scale`` in fp32, rounded
    once to bf16. Activation scales (``input_scale`` / ``activation_scale``), which only a quantised forward reads, are
    dropped; floats that were never quantised land as bf16. A source without a single fp8 tensor is refused (the result
    would be a plain copy reported as a conversion)."""
    _reject_in_place(src, dst)
    idx = CheckpointIndex(src)
    names = sorted(idx.weight_map)
    fp8 = [n for n in names if n.endswith("weight") and n + "_scale" in idx]
    if not fp8:
        raise ValueError(f"{src!r} holds no tensor with a static weight_scale beside it: nothing to dequantise")
    writer = StreamingShardWriter(dst)
    n_done = 0
    for name in names:
        if name.endswith(("weight_scale", "input_scale", "activation_scale")):
            continue
        t = idx.get(name)
        if name + "_scale" in idx:
            if t.dtype != torch.float8_e4m3fn:
                raise ValueError(f"{name} has a weight_scale but is {t.dtype}, not float8_e4m3fn")
            s = idx.get(name + "_scale").float().reshape(-1)
            if s.numel() == 1:
                full = s.reshape(())
            elif t.dim() == 3 and s.numel() == t.shape[0]:
                full = s.reshape(-1, 1, 1)
            else:
                raise ValueError(f"{name}_scale has {s.numel()} entries: expected one for the matrix"
                                 + (f" or one per expert ({t.shape[0]})" if t.dim() == 3 else ""))
            t = (t.float() * full).to(torch.bfloat16)
            n_done += 1
        elif t.is_floating_point() and t.dtype != torch.bfloat16:
            t = t.to(torch.bfloat16)
        writer.add(name, t)
    writer.finish()
    copy_side_files(src, dst)
    _as_plain_bf16_config(dst)
    return n_done


from halo_b200.ops.lowp import E2M1_VALUES as _E2M1, unpack_mxfp4_blocks  # noqa: E402


def dequant_mxfp4_experts(src: str, dst: str) -> int:
    """Releases whose expert banks are packed MXFP4 (the gpt-oss hub layout): ``<bank>_blocks`` and ``<bank>_scales``
    become ``<bank>`` in bf16. The packed form stores a bank as ``[E, out, G, 16]`` (the reduction axis blocked last);
    the bf16 form the family's loaders read is ``[E, in, out]``, so the unpacked bank is transposed. Everything else is
    copied as it is."""
    _reject_in_place(src, dst)
    idx = CheckpointIndex(src)
    names = sorted(idx.weight_map)
    packed = [n[:-len("_blocks")] for n in names if n.endswith("_blocks")]
    if not packed:
        raise ValueError(f"{src!r} holds no '<name>_blocks' tensor: nothing to dequantise")
    writer = StreamingShardWriter(dst)
    for name in names:
        if name.endswith("_scales") and name[:-len("_scales")] in packed:
            continue
        if name.endswith("_blocks"):
            base = name[:-len("_blocks")]
            if base + "_scales" not in idx:
                raise KeyError(f"{name} has no {base}_scales beside it")
            full = unpack_mxfp4_blocks(idx.get(name), idx.get(base + "_scales"))
            if full.dim() == 3:
                full = full.transpose(1, 2)
            writer.add(base, full.to(torch.bfloat16).contiguous())
            continue
        writer.add(name, idx.get(name))
    writer.finish()
    copy_side_files(src, dst)
    _as_plain_bf16_config(dst)
    return len(packed)


def export_block_fp8(src: str, dst: str, keep: list[str] | None = None) -> int:
    """bf16 matrices -> ``float8_e4m3fn`` with one fp32 ``weight_scale_inv`` per 128 x 128 block (the served-weights layout
    :func:`dequant_block_fp8` reads; inference engines load it directly)."""
    kept = [re.compile(p) for p in keep or []]
    idx = CheckpointIndex(src)
    writer = StreamingShardWriter(dst)
    n = 0
    for name in sorted(idx.weight_map):
        t = idx.get(name)
        if t.dim() != 2 or not name.endswith(".weight") or ALWAYS_KEPT.search(name) or any(p.search(name) for p in kept):
            writer.add(name, t)
            continue
        rows, cols = t.shape
        pr, pc = -(-rows // BLOCK) * BLOCK, -(-cols // BLOCK) * BLOCK
        padded = torch.zeros(pr, pc, dtype=torch.float32)
        padded[:rows, :cols] = t.float()
        blocks = padded.view(pr // BLOCK, BLOCK, pc // BLOCK, BLOCK)
        scale = (blocks.abs().amax(dim=(1, 3)) / lowp.E4M3_MAX).clamp(min=1e-12)              # [rows/128, cols/128]
        q = (blocks / scale[:, None, :, None]).clamp(-lowp.E4M3_MAX, lowp.E4M3_MAX).to(torch.float8_e4m3fn)
        writer.add(name, q.view(pr, pc)[:rows, :cols].contiguous())
        writer.add(name + "_scale_inv", scale)
        n += 1
    writer.finish()
    copy_side_files(src, dst)
    cfg_path = os.path.join(dst, "config.json")
    if os.path.isfile(cfg_path):
        cfg = json.load(open(cfg_path))
        cfg["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [BLOCK, BLOCK],
                                      "activation_scheme": "dynamic"}
        json.dump(cfg, open(cfg_path, "w"), indent=2)
    return n


def export(src: str, dst: str, fmt: str, keep: list[str] | None = None, layout: str = "block_scaled") -> int:
    """``layout``: ``block_scaled`` writes the framework's own manifest (``halo_lowp.json``); ``compressed-tensors`` also
    writes the ``quantization_config`` a serving engine's compressed-tensors loader reads."""
    if layout not in ("block_scaled", "compressed-tensors"):
        raise ValueError(f"unknown layout {layout!r}")
    if fmt not in lowp.FORMATS:
        raise ValueError(f"unknown format {fmt!r}; known: {lowp.FORMATS}")
    kept = [re.compile(p) for p in keep or []]
    idx = CheckpointIndex(src)
    writer = StreamingShardWriter(dst)
    n = 0
    quantized_modules, kept_modules = [], []
    for name in sorted(idx.weight_map):
        t = idx.get(name)
        plain = (t.dim() != 2 or not name.endswith(".weight") or ALWAYS_KEPT.search(name) or any(p.search(name) for p in kept)
                 or t.shape[1] % lowp.BLOCK_SIZE[fmt])
        if plain:
            writer.add(name, t)
            if t.dim() == 2 and name.endswith(".weight"):
                kept_modules.append(name[:-len(".weight")])
            continue
        quantized_modules.append(name[:-len(".weight")])
        q = lowp.quantize(t, fmt)
        data = q.data.view(torch.uint8) if q.data.dtype == torch.float8_e4m3fn else q.data       # bytes either way
        scales = q.scales.view(torch.uint8) if q.scales.dtype == torch.float8_e4m3fn else q.scales
        writer.add(name, data)
        writer.add(name + "_scale", scales)
        if q.global_scale is not None:
            writer.add(name + "_global_scale", q.global_scale.reshape(1).float())
        n += 1
    writer.finish()
    copy_side_files(src, dst)
    json.dump({"format": fmt, "block_size": lowp.BLOCK_SIZE[fmt], "quantized_tensors": n},
              open(os.path.join(dst, "halo_lowp.json"), "w"), indent=2)
    if layout == "compressed-tensors":
        from .compressed_tensors_layout import quantization_config

        cfg_path = os.path.join(dst, "config.json")
        cfg = json.load(open(cfg_path)) if os.path.isfile(cfg_path) else {}
        cfg["quantization_config"] = quantization_config(fmt, quantized_modules, kept_modules)
        json.dump(cfg, open(cfg_path, "w"), indent=2)
    return n


def dequant(src: str, dst: str) -> int:
    meta = json.load(open(os.path.join(src, "halo_lowp.json")))
    fmt = meta["format"]
    idx = CheckpointIndex(src)
    writer = StreamingShardWriter(dst)
    n = 0
    for name in sorted(idx.weight_map):
        if name.endswith(("_scale", "_global_scale")) and name.rsplit("_scale", 1)[0].rsplit("_global", 1)[0] in idx:
            continue
        t = idx.get(name)
        if name + "_scale" in idx:
            scales = idx.get(name + "_scale")
            data = t.view(torch.float8_e4m3fn) if fmt == "mxfp8" else t
            if fmt == "nvfp4":
                scales = scales.view(torch.float8_e4m3fn)
            gs = idx.get(name + "_global_scale")[0] if name + "_global_scale" in idx else None
            t = lowp.dequantize(lowp.BlockScaledTensor(data, scales, fmt, gs), torch.bfloat16)
            n += 1
        writer.add(name, t)
    writer.finish()
    copy_side_files(src, dst)
    return n


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    for cmd in ("dequant-block-fp8", "dequant", "dequant-static-fp8", "dequant-mxfp4-experts"):
        p = sub.add_parser(cmd)
        p.add_argument("src")
        p.add_argument("dst")
    p = sub.add_parser("export-block-fp8")
    p.add_argument("src")
    p.add_argument("dst")
    p.add_argument("--keep", nargs="*", default=[])
    p = sub.add_parser("export")
    p.add_argument("src")
    p.add_argument("dst")
    p.add_argument("--format", required=True, choices=list(lowp.FORMATS))
    p.add_argument("--keep", nargs="*", default=[])
    p.add_argument("--layout", default="block_scaled", choices=["block_scaled", "compressed-tensors"])
    args = ap.parse_args(argv)
    if args.cmd == "dequant-block-fp8":
        n = dequant_block_fp8(args.src, args.dst)
    elif args.cmd == "dequant":
        n = dequant(args.src, args.dst)
    elif args.cmd == "dequant-static-fp8":
        n = dequant_static_fp8(args.src, args.dst)
    elif args.cmd == "dequant-mxfp4-experts":
        n = dequant_mxfp4_experts(args.src, args.dst)
    elif args.cmd == "export-block-fp8":
        n = export_block_fp8(args.src, args.dst, args.keep)
    else:
        n = export(args.src, args.dst, args.format, args.keep, args.layout)
    print(f"{args.cmd}: {n} tensors converted into {args.dst}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
