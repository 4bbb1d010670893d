"""Config parser, argument dataclasses, parallelism rules and rank layouts (CPU)."""

import pytest

from halo_b200.config_validation import ConfigError
from halo_b200.configs.arguments import (DataArguments, ModelArguments, ParallelismArguments, SFTArguments,
                                         TrainingArguments)
from halo_b200.configs.parser import ArgumentParser, expand_output_dir
from halo_b200.parallel import layout as L
from halo_b200.parallel.config import ParallelismConfig
from halo_b200.parallel.rules import SUPPORTED_AXIS_SETS, reject_model_layout


def _parser():
    return ArgumentParser(ModelArguments, DataArguments, TrainingArguments, ParallelismArguments, SFTArguments)


def test_yaml_then_cli_override(tmp_path):
    y = tmp_path / "c.yaml"
    y.write_text("model_preset: tiny-moe\nlearning_rate: 2.0e-4\nexpert_parallel_size: 2\npipeline_split: [2, 2]\n")
    m, d, t, p, s = _parser().parse([str(y), "--learning_rate=1e-3", "--max_steps=5"])
    assert t.learning_rate == 1e-3 and t.max_steps == 5 and p.expert_parallel_size == 2
    assert p.pipeline_split == [2, 2] and m.init_from_scratch and t.bf16 is True


def test_unknown_retired_and_container_keys(tmp_path):
    with pytest.raises(ConfigError, match="Did you mean"):
        _parser().parse(["--model_preset=tiny-moe", "--learning_rat=1"])
    with pytest.raises(ConfigError, match="retired"):
        _parser().parse(["--model_preset=tiny-moe", "--use_liger_kernel=true"])
    with pytest.raises(ConfigError, match="YAML"):
        _parser().parse(["--model_preset=tiny-moe", "--pipeline_split=[1,3]"])
    with pytest.raises(ConfigError, match="one of"):
        _parser().parse(["--model_preset=tiny-moe", "--pipeline_schedule=zigzag"])


def test_output_dir_pattern():
    assert expand_output_dir("runs/%Y", now=0).startswith("runs/19")
    assert expand_output_dir("runs/fixed") == "runs/fixed"


def test_allowlist_has_eleven_sets_and_refusals_explain():
    assert len(SUPPORTED_AXIS_SETS) == 11
    for kw, needle in ((dict(tp_size=2, cp_size=2), "TP partners"), (dict(expert_tp_size=2, cp_size=2), "same tokens"),
                       (dict(pp_size=2, cp_size=2), "too small")):
        with pytest.raises(ConfigError, match=needle):
            ParallelismConfig(world_size=8, global_rank=0, **kw)


@pytest.mark.parametrize("world,kw,dp", [
    (8, dict(), 8), (8, dict(ep_size=8), 8), (8, dict(ep_size=4, expert_tp_size=2), 4), (8, dict(tp_size=2), 4),
    (8, dict(cp_size=2), 4), (8, dict(ep_size=8, cp_size=2), 4), (8, dict(ep_size=8, tp_size=2), 4),
    (8, dict(pp_size=2, ep_size=4, nvlink_domain_size=4), 4), (16, dict(ep_size=16, gpus_per_node=8), 16),
])
def test_supported_layouts_and_data_parallel_width(world, kw, dp):
    for rank in range(world):
        pc = ParallelismConfig(world_size=world, global_rank=rank, **kw)
        assert pc.data_parallel_size == dp
        assert rank in pc.ep_group_ranks() and rank in pc.dp_group_ranks() and rank in pc.pp_chain_ranks()


def test_groups_partition_the_world():
    pc = ParallelismConfig(world_size=16, global_rank=0, ep_size=4, expert_tp_size=2, gpus_per_node=8)
    for kind in ("ep_group", "dispatch_group", "expert_tp_group", "expert_replica", "dp_group"):
        groups = pc.all_groups(kind)
        flat = sorted(r for g in groups for r in g)
        assert flat == list(range(16)), kind
    assert pc.all_groups("expert_tp_group")[0] == [0, 4]
    assert pc.all_groups("dispatch_group")[0] == [0, 1, 2, 3]


def test_layouts_at_scale():
    lay = L.StridedLayout(4096, 1024, 72 * 0 + 8)
    seen = set()
    for g in range(lay.num_groups):
        ranks = lay.group_ranks(g)
        assert len(ranks) == 1024 and not (seen & set(ranks))
        seen |= set(ranks)
        for pos, r in enumerate(ranks):
            assert lay.locate(r) == (pos, g)
    assert len(seen) == 4096
    blk = L.BlockLayout(1024, 8, 8)
    assert blk.locate(731) == (3, 91) and blk.replica_ranks(3)[91] == 731


def test_model_dependent_refusals():
    from halo_b200.models.config import moe_30b_a3b_config, dense_9b_config

    with pytest.raises(ConfigError, match="not divisible"):
        reject_model_layout(ParallelismConfig(world_size=6, global_rank=0, ep_size=6, gpus_per_node=6), moe_30b_a3b_config())
    with pytest.raises(ConfigError, match="without routed experts"):
        reject_model_layout(ParallelismConfig(world_size=8, global_rank=0, ep_size=8), dense_9b_config())
    reject_model_layout(ParallelismConfig(world_size=8, global_rank=0, tp_size=2), dense_9b_config())


def test_prepared_dataset_round_trip_and_coordinated_cache(tmp_path):
    import json

    import numpy as np

    from halo_b200.data import preprocessed as pp

    src = tmp_path / "docs.jsonl"
    rng = np.random.default_rng(0)
    with open(src, "w") as f:
        for _ in range(40):
            f.write(json.dumps({"input_ids": rng.integers(0, 100, size=int(rng.integers(5, 60))).tolist()}) + "\n")
    out = str(tmp_path / "prepared")
    assert pp.main([str(src), out, "--row-len", "128"]) == 0
    meta = pp.read_metadata(out)
    rows0, rows1 = pp.load_rows(out, 0, 2, expect_row_len=128), pp.load_rows(out, 1, 2)
    assert len(rows0) + len(rows1) == meta["n_rows"] and all(r.n_tokens == 128 for r in rows0 + rows1)
    assert rows0[0].cu_seqlens[0] == 0 and rows0[0].cu_seqlens[-1] == 128
    import pytest

    with pytest.raises(ValueError, match="packed to 128"):
        pp.load_rows(out, expect_row_len=256)
    with pytest.raises(FileNotFoundError):
        pp.read_metadata(str(tmp_path))
    calls = []

    def build(d):
        calls.append(d)
        open(d + "/artifact", "w").write("x")

    d1 = pp.coordinated_cache(str(tmp_path / "cache"), ["a", 1], build)
    d2 = pp.coordinated_cache(str(tmp_path / "cache"), ["a", 1], build)
    d3 = pp.coordinated_cache(str(tmp_path / "cache"), ["a", 1], build, rank=1, wait_seconds=1)     # found: no wait
    assert d1 == d2 == d3 and len(calls) == 1
    with pytest.raises(TimeoutError):
        pp.coordinated_cache(str(tmp_path / "cache"), ["b"], build, rank=1, wait_seconds=0.3, poll_seconds=0.05)


def test_freeze_patterns_preflight_and_collators(tmp_path):
    import dataclasses

    import numpy as np
    import pytest
    import torch

    from halo_b200.checkpoint.preflight import checkpoint_bytes, require_free_space
    from halo_b200.data import collators
    from halo_b200.models.config import PRESETS
    from halo_b200.models.freeze import apply_freeze_patterns
    from halo_b200.models.qwen3 import build_model

    model = build_model(dataclasses.replace(PRESETS["tiny-moe"](), num_hidden_layers=2), device="cpu", dtype=torch.float32)
    stats = apply_freeze_patterns(model, freeze=["embed_tokens", r"layers\.0\."])
    assert not model.embed_tokens.requires_grad and not model.layers[0].self_attn.o_proj.requires_grad
    assert model.layers[1].self_attn.o_proj.requires_grad and stats["frozen"] > 0 and stats["trainable"] > 0
    with pytest.raises(ValueError, match="matches no parameter"):
        apply_freeze_patterns(model, freeze=["no_such_tensor"])
    apply_freeze_patterns(model, train_only=[r"mlp\.gate$"])
    assert sum(p.requires_grad for p in model.parameters()) == 2
    need = checkpoint_bytes(model, with_optimizer=False)
    assert need == sum(p.numel() * 4 for p in model.parameters())
    assert require_free_space(str(tmp_path / "new" / "dir"), 1024) > 0
    with pytest.raises(OSError, match="GiB are free"):
        require_free_space(str(tmp_path), 1 << 60)
    docs = [np.arange(5), np.arange(3)]
    assert collators.padding_free(docs).n_tokens == 8
    fs = collators.fixed_shape(docs, 16)
    assert fs.n_tokens == 16 and fs.cu_seqlens.tolist() == [0, 5, 8, 16] and fs.n_scored == 6
    with pytest.raises(ValueError):
        collators.fixed_shape(docs, 6)
    pb = collators.padded(docs, pad_token_id=9, pad_to_multiple_of=4)
    assert pb["input_ids"].shape == (2, 8) and pb["attention_mask"].sum().item() == 8 and pb["input_ids"][1, 3].item() == 9
    assert pb["labels"][0, :4].tolist() == [1, 2, 3, 4] and pb["labels"][0, 4].item() == -100


def test_reference_recipe_converts_and_parses(tmp_path):
    import dataclasses

    import yaml

    from halo_b200.configs import arguments as A
    from halo_b200.configs import convert_recipe
    from halo_b200.configs.parser import ArgumentParser

    fields = set()
    for name in dir(A):
        c = getattr(A, name)
        if dataclasses.is_dataclass(c) and isinstance(c, type):
            fields |= {f.name for f in dataclasses.fields(c)}
    assert not (convert_recipe.KEPT - fields) and not ({v[0] for v in convert_recipe.RENAMED.values()} - fields)

    data = tmp_path / "train.jsonl"
    data.write_text('{"messages": []}\n')
    recipe = {"model_name_or_path": "/models/qwen3-30b-a3b", "dataset": [str(data)], "conversation_field": "messages",
              "assistant_message_template": "<|im_start|>assistant\n", "use_peft": True, "lora_r": 64, "lora_alpha": 128,
              "lora_target_modules": ["q_proj", "v_proj"], "per_device_train_batch_size": 4, "gradient_accumulation_steps": 4,
              "gradient_checkpointing_kwargs": {"use_reentrant": False}, "learning_rate": 1e-4, "lr_scheduler_type": "cosine",
              "warmup_steps": 32, "max_length": 4096, "packing": True, "output_dir": "checkpoints/x", "eval_strategy": "steps",
              "eval_steps": 500, "save_total_limit": 3, "save_only_model": True, "logging_steps": 1, "logging_first_step": True,
              "report_to": "none", "dataloader_num_workers": 4, "attn_implementation": "flash_attention_4", "expert_parallel_size": 8,
              "moe_balancing": "bias_update", "fp32_grad_reduce": True}
    src, dst = tmp_path / "ref.yaml", tmp_path / "ours.yaml"
    src.write_text(yaml.safe_dump(recipe))
    assert convert_recipe.main([str(src), str(dst)]) == 0
    text = dst.read_text()
    assert "launch sft" in text and "dropped attn_implementation" in text and "dataloader_num_workers -> num_proc" in text
    parsed = ArgumentParser(A.ModelArguments, A.DataArguments, A.TrainingArguments, A.ParallelismArguments, A.SFTArguments).parse([str(dst)])
    assert parsed[0].lora_r == 64 and parsed[1].dataset_path == str(data) and parsed[1].completion_only_loss and parsed[1].num_proc == 4
    assert parsed[3].expert_parallel_size == 8
    src.write_text(yaml.safe_dump({**recipe, "use_vllm": True, "images_field": "images", "num_generations": 8}))
    with pytest.raises(ValueError, match="images_field"):
        convert_recipe.main([str(src), str(dst)])
    assert convert_recipe.main([str(src), str(dst), "--lenient"]) == 0 and "NOT CONVERTED images_field" in dst.read_text()
    assert "launch grpo" in dst.read_text() and "dropped use_vllm: no generation server: add rollout_gpus" in dst.read_text()
