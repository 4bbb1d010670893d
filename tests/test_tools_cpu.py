"""Offline checkpoint tools, expert layout conversions, head transform, selection bias (CPU)."""

import json
import os

import pytest
import torch

from halo_b200.checkpoint.load import CheckpointIndex, from_pretrained
from halo_b200.checkpoint.save import save_model
from halo_b200.checkpoint.tools import convert_dtype, merge_models, patch_vocab, relayout_experts
from halo_b200.models import moe_families as mf
from halo_b200.models.config import PRESETS
from halo_b200.models.head_transform import HeadTransform, chunked_cross_entropy
from halo_b200.models.qwen3 import build_model
from halo_b200.ops.moe import router_topk_reference


def _tiny(tmp_path, seed, name):
    model = build_model(PRESETS["tiny-moe"](), device="cpu", dtype=torch.float32, seed=seed)
    d = str(tmp_path / name)
    save_model(model, d, save_dtype=None)
    return model, d


def test_layout_round_trips_every_kind():
    E, F, H = 4, 6, 8
    gu, dn = torch.randn(E, 2 * F, H), torch.randn(E, H, F)
    for kind in mf.LAYOUT_KINDS:
        back = mf.to_runtime_banks(kind, mf.from_runtime_banks(kind, gu, dn), E)
        assert torch.equal(back[0], gu) and torch.equal(back[1], dn), kind


def test_family_registry_refuses_unbuilt_decoders():
    assert mf.require_runnable("qwen3_moe").layout == mf.SEPARATE_GLU
    assert mf.require_runnable("gpt_oss").layout == mf.INTERLEAVED_GLU
    with pytest.raises(NotImplementedError, match="latent attention"):
        mf.require_runnable("deepseek_v4")
    with pytest.raises(KeyError):
        mf.family_spec("no_such_family")
    assert len(mf.families()) >= 18


def test_convert_and_merge_tools(tmp_path):
    a_model, a = _tiny(tmp_path, 0, "a")
    b_model, b = _tiny(tmp_path, 1, "b")
    out = str(tmp_path / "bf16")
    assert convert_dtype.main([a, out, "--dtype", "bfloat16"]) == 0
    idx = CheckpointIndex(out)
    assert idx.get("model.norm.weight").dtype == torch.bfloat16
    lin = str(tmp_path / "lin")
    merge_models.main([a, b, "--out", lin, "--method", "linear", "--weights", "1", "3"])
    name = "model.layers.0.self_attn.o_proj.weight"
    want = 0.25 * CheckpointIndex(a).get(name) + 0.75 * CheckpointIndex(b).get(name)
    assert torch.allclose(CheckpointIndex(lin).get(name), want, atol=1e-6)
    sl = str(tmp_path / "slerp")
    merge_models.main([a, b, "--out", sl, "--method", "slerp", "--t", "0.0"])
    assert torch.allclose(CheckpointIndex(sl).get(name), CheckpointIndex(a).get(name), atol=1e-5)
    ti = str(tmp_path / "ties")
    merge_models.main([a, a, "--out", ti, "--method", "ties", "--base", b, "--density", "1.0"])
    assert torch.allclose(CheckpointIndex(ti).get(name), CheckpointIndex(a).get(name), atol=1e-5)
    merged = from_pretrained(lin, device="cpu", dtype=torch.float32)     # the merge is a loadable checkpoint
    assert merged.cfg.num_experts == a_model.cfg.num_experts


def test_relayout_and_vocab_patch(tmp_path):
    model, a = _tiny(tmp_path, 0, "a")
    fused = str(tmp_path / "fused")
    relayout_experts.main([a, fused, "--from", "SEPARATE_GLU", "--to", "FUSED"])
    assert "model.layers.0.mlp.experts.gate_up_proj" in CheckpointIndex(fused).weight_map
    back = str(tmp_path / "back")
    relayout_experts.main([fused, back, "--from", "FUSED", "--to", "SEPARATE_GLU"])
    ia, ib = CheckpointIndex(a), CheckpointIndex(back)
    assert sorted(ia.weight_map) == sorted(ib.weight_map)
    for k in ia.weight_map:
        assert torch.equal(ia.get(k), ib.get(k)), k
    grown = str(tmp_path / "grown")
    v = model.cfg.vocab_size
    patch_vocab.main([a, grown, "--vocab-size", str(v + 16)])
    e = CheckpointIndex(grown).get("model.embed_tokens.weight")
    assert e.shape[0] == v + 16 and torch.allclose(e[-1], e[:v].mean(0), atol=1e-6)
    assert json.load(open(os.path.join(grown, "config.json")))["vocab_size"] == v + 16


def test_head_transform_matches_plain_cross_entropy_and_softcap_bounds_logits():
    torch.manual_seed(0)
    h, w, y = torch.randn(33, 16), torch.randn(50, 16), torch.randint(0, 50, (33,))
    plain = torch.nn.functional.cross_entropy(h @ w.t(), y)
    assert torch.allclose(chunked_cross_entropy(h, w, y, HeadTransform(), chunk_rows=8), plain, atol=1e-5)
    t = HeadTransform(logit_scale=2.0, softcap=5.0, vocab_cut=40)
    assert t.apply(h @ t.weight_view(w).t()).abs().max() <= 5.0 and not t.fusable


def test_selection_bias_changes_ranking_not_weights():
    torch.manual_seed(0)
    logits = torch.randn(64, 32)
    idx0, w0 = router_topk_reference(logits, 4, False)
    bias = torch.zeros(32)
    bias[7] = 10.0                                      # expert 7 is always selected now
    idx1, w1 = router_topk_reference(logits, 4, False, bias)
    assert bool((idx1 == 7).any(-1).all())
    probs = torch.softmax(logits, -1)
    assert torch.allclose(w1, probs.gather(-1, idx1.long()))      # weights are the unbiased probabilities


def test_trace_report_groups_kernels_and_measures_overlap(tmp_path):
    import gzip
    import json

    from halo_b200.diagnostics import trace_report

    def ev(name, ts, dur, tid=7, cat="kernel"):
        return {"ph": "X", "cat": cat, "name": name, "ts": ts, "dur": dur, "pid": 0, "tid": tid}

    events = [ev("gemm_bf16_kernel<0,0>", 0, 100), ev("gemm_bf16_kernel<0,0>", 100, 100), ev("attn_fwd_kernel", 200, 50),
              ev("ncclDevKernel_AllReduce", 150, 100, tid=9), ev("rmsnorm_fwd_kernel<1,32>", 300, 10),
              {"ph": "X", "cat": "cpu_op", "name": "aten::mm", "ts": 0, "dur": 500, "pid": 1, "tid": 1}]
    path = tmp_path / "trace.json.gz"
    with gzip.open(path, "wt") as f:
        json.dump({"traceEvents": events}, f)
    rep = trace_report.summarise(trace_report.load_events(str(path)))
    assert rep["launches"] == 5 and rep["device_time_us"] == 360.0
    assert rep["kernels"][0]["name"].startswith("gemm_bf16") and rep["kernels"][0]["launches"] == 2
    assert rep["families"] == {"gemm": 200.0, "collectives": 100.0, "attention": 50.0, "element-wise": 10.0}
    assert rep["span_us"] == 310.0 and rep["busy_us"] == 260.0 and rep["overlap_us"] == 100.0      # the all-reduce ran beside compute
    assert trace_report.main([str(path), "--top", "3"]) == 0


def test_pipeline_stage_directories_merge_into_one_loadable_checkpoint(tmp_path):
    """Two nodes, each holding only its own stage's shard files (node 0 also the index and config): the merge tool
    unions them, and refuses when a node's directory is missing or stages overlap."""
    import json
    import os
    import shutil

    from halo_b200.checkpoint.tools import merge_pp_stages

    model, full = _tiny(tmp_path, 0, "whole")
    idx = CheckpointIndex(full)
    names = sorted(idx.weight_map)
    half = len(names) // 2
    node0, node1 = tmp_path / "node0", tmp_path / "node1"
    from safetensors.torch import save_file

    node0.mkdir(), node1.mkdir()
    save_file({n: idx.get(n).contiguous() for n in names[:half]}, str(node0 / "model-stage000-00001.safetensors"))
    save_file({n: idx.get(n).contiguous() for n in names[half:]}, str(node1 / "model-stage001-00001.safetensors"))
    shutil.copy(os.path.join(full, "config.json"), node0 / "config.json")
    json.dump({"metadata": {}, "weight_map": {n: "x" for n in names}}, open(node0 / "model.safetensors.index.json", "w"))
    out = str(tmp_path / "merged")
    assert merge_pp_stages.main([str(node0), str(node1), "--out", out]) == 0
    merged = from_pretrained(out, device="cpu", dtype=torch.float32)
    for (n, p), (_, q) in zip(model.named_parameters(), merged.named_parameters()):
        assert torch.equal(p, q), n
    with pytest.raises(ValueError, match="in none of the directories"):
        merge_pp_stages.merge([str(node0)], str(tmp_path / "partial"))
    shutil.copy(node0 / "model-stage000-00001.safetensors", node1 / "model-stage009-00001.safetensors")
    with pytest.raises(ValueError, match="stages overlap"):
        merge_pp_stages.merge([str(node0), str(node1)], str(tmp_path / "overlap"))


def test_compressed_tensors_block_names_the_quantised_modules(tmp_path):
    import json
    import os
    import re

    from halo_b200.checkpoint.tools import lowp_convert
    from halo_b200.checkpoint.tools.compressed_tensors_layout import module_targets, quantization_config

    targets = module_targets(["model.layers.0.self_attn.q_proj", "model.layers.11.self_attn.q_proj",
                              "model.layers.3.mlp.experts.17.down_proj"])
    assert targets == [r"re:model\.layers\.\d+\.mlp\.experts\.\d+\.down_proj", r"re:model\.layers\.\d+\.self_attn\.q_proj"]
    cfg = quantization_config("nvfp4", ["model.layers.1.self_attn.q_proj"], ["model.layers.0.self_attn.q_proj", "lm_head"])
    assert cfg["ignore"] == ["model.layers.0.self_attn.q_proj"]          # a kept module the generalised pattern would sweep in
    assert cfg["config_groups"]["group_0"]["weights"]["group_size"] == 16
    _, ckpt = _tiny(tmp_path, 0, "src")
    out = str(tmp_path / "ct")
    assert lowp_convert.main(["export", ckpt, out, "--format", "mxfp8", "--keep", r"layers\.0\.", "--layout", "compressed-tensors"]) == 0
    qc = json.load(open(os.path.join(out, "config.json")))["quantization_config"]
    assert qc["quant_method"] == "compressed-tensors" and qc["format"] == "mxfp8-quantized"
    pats = [re.compile(t[3:] + "$") for t in qc["config_groups"]["group_0"]["targets"]]
    manifest = json.load(open(os.path.join(out, "halo_lowp.json")))
    assert manifest["quantized_tensors"] > 0
    idx = CheckpointIndex(out)
    for name in idx.weight_map:
        if name.endswith(".weight_scale"):
            module = name[:-len(".weight_scale")]
            assert any(p.match(module) for p in pats) and module not in qc["ignore"], module
    assert all("layers.0." in m for m in qc["ignore"]) and qc["ignore"]


def test_reattach_vision(tmp_path):
    """A trained text tower goes back into its multimodal wrapper: trained tensors under the wrapper's names, the vision
    tower streamed back, the composite config regrafted; mismatches are refused by name."""
    import json

    import pytest
    import torch
    from safetensors.torch import save_file

    from halo_b200.checkpoint.load import CheckpointIndex
    from halo_b200.checkpoint.tools import reattach_vision as R

    torch.manual_seed(0)
    base = {"model.language_model.embed_tokens.weight": torch.randn(10, 4), "model.language_model.layers.0.mlp.down_proj.weight": torch.randn(4, 8),
            "model.language_model.norm.weight": torch.ones(4), "lm_head.weight": torch.randn(10, 4),
            "model.visual.patch_embed.weight": torch.randn(6, 3), "model.multi_modal_projector.linear.weight": torch.randn(4, 6)}
    trained = {"model.embed_tokens.weight": torch.randn(10, 4), "model.layers.0.mlp.down_proj.weight": torch.randn(4, 8),
               "model.norm.weight": torch.full((4,), 2.0), "lm_head.weight": torch.randn(10, 4),
               "model.mtp.proj.weight": torch.randn(4, 8)}
    for name, tensors, cfg in (("base", base, {"model_type": "wrapper_vl", "vision_config": {"depth": 2}, "text_config": {"model_type": "wrapper_text", "hidden_size": 4}}),
                               ("export", trained, {"model_type": "qwen3", "hidden_size": 4, "architectures": ["Qwen3ForCausalLM"], "rope_theta": 5.0})):
        (tmp_path / name).mkdir()
        save_file(tensors, str(tmp_path / name / "model.safetensors"))
        (tmp_path / name / "config.json").write_text(json.dumps(cfg))
    (tmp_path / "base" / "preprocessor_config.json").write_text("{}")
    assert R.main([str(tmp_path / "export"), str(tmp_path / "base"), str(tmp_path / "out")]) == 0
    out = CheckpointIndex(str(tmp_path / "out"))
    assert sorted(out.weight_map) == sorted(list(base) + ["model.language_model.mtp.proj.weight"])
    assert torch.equal(out.get("model.language_model.norm.weight"), trained["model.norm.weight"])
    assert torch.equal(out.get("lm_head.weight"), trained["lm_head.weight"])
    assert torch.equal(out.get("model.visual.patch_embed.weight"), base["model.visual.patch_embed.weight"])
    assert torch.equal(out.get("model.language_model.mtp.proj.weight"), trained["model.mtp.proj.weight"])
    cfg = json.load(open(tmp_path / "out" / "config.json"))
    assert cfg["model_type"] == "wrapper_vl" and cfg["vision_config"] == {"depth": 2}
    assert cfg["text_config"] == {"model_type": "wrapper_text", "hidden_size": 4, "rope_theta": 5.0}
    assert (tmp_path / "out" / "preprocessor_config.json").is_file()
    # refusals
    with pytest.raises(ValueError, match="not text-only"):
        R.plan(list(trained) + ["model.visual.x"], list(base))
    with pytest.raises(ValueError, match="not a multimodal checkpoint"):
        R.plan(list(trained), [n for n in base if "visual" not in n and "projector" not in n])
    with pytest.raises(ValueError, match="names no tensor of the base's text tower"):
        R.plan(list(trained) + ["model.layers.1.mlp.down_proj.weight"], list(base))
    with pytest.raises(ValueError, match="lacks 1 tensors"):
        R.plan([n for n in trained if "norm" not in n], list(base))
    wrong = dict(trained)
    wrong["model.layers.0.mlp.down_proj.weight"] = torch.randn(4, 16)
    (tmp_path / "wrong").mkdir()
    save_file(wrong, str(tmp_path / "wrong" / "model.safetensors"))
    (tmp_path / "wrong" / "config.json").write_text("{}")
    with pytest.raises(ValueError, match="a base of another size"):
        R.reattach(str(tmp_path / "wrong"), str(tmp_path / "base"), str(tmp_path / "out2"))
    with pytest.raises(ValueError, match="one of the inputs"):
        R.reattach(str(tmp_path / "export"), str(tmp_path / "base"), str(tmp_path / "base"))
