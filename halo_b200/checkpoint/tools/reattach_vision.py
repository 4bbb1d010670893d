"""Put a trained text tower back into the multimodal checkpoint it was taken from.

A multimodal release (a text tower inside a wrapper that also holds a vision tower and a projector) is trained here as
its text model alone. This tool writes the composite again: the wrapper's text-tower tensors are replaced by the trained
ones (re-prefixed onto the wrapper's names), every other tensor of the base streams back in unchanged, and the composite
``config.json`` keeps the base's vision part with the trained text part in place of its ``text_config``.

    python -m halo_b200.checkpoint.tools.reattach_vision <text_export> <multimodal_base> <dst>

Refused by name: an export that is not text-only; an export whose tensors name no module of the base's text tower (a head
the run added, such as a multi-token-prediction block, is carried over under the wrapper's prefix and reported); a base
whose text tower has another shape (what streams back from it was built against its own tower); writing over an input.
(The role of halo/checkpoint/tools/vision_reattach.py.)"""

from __future__ import annotations

import argparse
import json
import os
import sys

from ._io import CheckpointIndex, StreamingShardWriter, copy_side_files

_EMBED = "embed_tokens.weight"
_MEDIA_MARKS = ("vision", "visual", "audio", "image", "multi_modal_projector", "mm_projector")
_ADDED_HEAD_MARKS = ("mtp.", "mtp_head.", ".mtp")


def text_prefix(names) -> str:
    """What precedes ``embed_tokens.weight`` in a checkpoint's names: ``model.`` for a text model,
    ``model.language_model.`` / ``language_model.model.`` for a wrapper."""
    hits = [n for n in names if n.endswith(_EMBED)]
    if len(hits) != 1:
        raise ValueError(f"expected exactly one '*{_EMBED}' tensor, found {hits}")
    return hits[0][:-len(_EMBED)]


def is_media_name(name: str) -> bool:
    return any(mark in name for mark in _MEDIA_MARKS)


def plan(export_names, base_names) -> tuple[dict[str, str], list[str], list[str]]:
    """``(export name -> composite name, carried extras, base names that stream back)``."""
    media = [n for n in export_names if is_media_name(n)]
    if media:
        raise ValueError(f"the export is not text-only: it holds {media[0]!r} (and {len(media) - 1} more)")
    if not any(is_media_name(n) for n in base_names):
        raise ValueError("the base holds no vision / projector tensors: it is not a multimodal checkpoint")
    ep, bp = text_prefix(export_names), text_prefix(base_names)
    base_set = set(base_names)
    mapping, extras = {}, []
    for n in export_names:
        if n.startswith(ep):
            target = bp + n[len(ep):]
        else:
            target = n                                     # lm_head and other top-level tensors keep their names
        if target not in base_set:
            if any(mark in n for mark in _ADDED_HEAD_MARKS):
                extras.append(target)                      # a head the run trained: carried under the wrapper's prefix
            else:
                raise ValueError(f"{n!r} of the export names no tensor of the base's text tower ({target!r}): the export and "
                                 "the base are not the same architecture")
        mapping[n] = target
    replaced = set(mapping.values())
    missing = [n for n in base_names if n.startswith(bp) and not is_media_name(n) and n not in replaced]
    if missing:
        raise ValueError(f"the export lacks {len(missing)} tensors of the base's text tower (first: {missing[0]!r})")
    kept = [n for n in base_names if n not in replaced]
    return mapping, extras, kept


def composite_config(base_cfg: dict, export_cfg: dict) -> dict:
    """The base's composite config with the trained text configuration in place of its ``text_config``."""
    if "text_config" not in base_cfg:
        raise ValueError("the base's config.json has no text_config: it does not describe a wrapper around a text tower")
    out = dict(base_cfg)
    text = {k: v for k, v in export_cfg.items() if k not in ("architectures", "transformers_version", "auto_map", "quantization_config")}
    text["model_type"] = base_cfg["text_config"].get("model_type", text.get("model_type"))
    out["text_config"] = text
    if "tie_word_embeddings" in export_cfg:
        out["tie_word_embeddings"] = export_cfg["tie_word_embeddings"]
    return out


def reattach(export_dir: str, base_dir: str, dst: str) -> dict:
    for d in (export_dir, base_dir):
        if os.path.realpath(d) == os.path.realpath(dst):
            raise ValueError("the output directory is one of the inputs: the writer would delete the shards it is reading")
    export, base = CheckpointIndex(export_dir), CheckpointIndex(base_dir)
    mapping, extras, kept = plan(sorted(export.weight_map), sorted(base.weight_map))
    incoming = {target: name for name, target in mapping.items()}
    writer = StreamingShardWriter(dst)
    for target in sorted(set(kept) | set(incoming)):
        if target in incoming:
            t = export.get(incoming[target])
            if target in base.weight_map:
                want = tuple(base.get(target).shape)
                if tuple(t.shape) != want:
                    raise ValueError(f"{target!r} is {tuple(t.shape)} in the export and {want} in the base: a base of another "
                                     "size in the same family; re-attach to the checkpoint the text tower was taken from")
            writer.add(target, t)
        else:
            writer.add(target, base.get(target))
    writer.finish()
    copy_side_files(base_dir, dst)                         # the processor / tokenizer files of the multimodal release
    for name in ("preprocessor_config.json", "processor_config.json", "video_preprocessor_config.json"):
        p = os.path.join(base_dir, name)
        if os.path.isfile(p):
            import shutil

            shutil.copy2(p, os.path.join(dst, name))
    base_cfg = json.load(open(os.path.join(base_dir, "config.json")))
    export_cfg = json.load(open(os.path.join(export_dir, "config.json")))
    json.dump(composite_config(base_cfg, export_cfg), open(os.path.join(dst, "config.json"), "w"), indent=2)
    return {"replaced": len(mapping) - len(extras), "carried": extras, "streamed_back": len(kept)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("text_export")
    ap.add_argument("multimodal_base")
    ap.add_argument("dst")
    a = ap.parse_args(argv)
    r = reattach(a.text_export, a.multimodal_base, a.dst)
    extra = f", {len(r['carried'])} added-head tensors carried ({r['carried'][0]} ...)" if r["carried"] else ""
    print(f"{r['replaced']} text-tower tensors replaced, {r['streamed_back']} tensors streamed back from the base{extra}: {a.dst}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
