"""Data sources on CPU: chat rendering finds the assistant spans by prefix rendering (and notices templates that rewrite
history), corpus mixes keep their ratios on every prefix and resume, shards and the replica identity check, best-fit
packing."""

import numpy as np
import pytest

from halo_b200.data.chat_render import completion_spans, render_conversation
from halo_b200.data.sources import CorpusMix, assert_replicas_identical, best_fit_rows, data_digest, shard_for_rank
from tests.common.gloo import run_gloo_ranks


class WordTokenizer:
    """Whitespace words are tokens; the template wraps turns in role markers."""

    chat_template = "yes"

    def __init__(self, drop_old_reasoning=False):
        self.vocab, self.drop = {}, drop_old_reasoning

    def _ids(self, text):
        return [self.vocab.setdefault(w, len(self.vocab)) for w in text.split()]

    def apply_chat_template(self, messages, add_generation_prompt=False, tokenize=True, tools=None):
        parts = []
        last_user = max((i for i, m in enumerate(messages) if m["role"] == "user"), default=-1)
        for i, m in enumerate(messages):
            content = m["content"]
            if self.drop and m["role"] == "assistant" and i < last_user:
                content = content.split("</think>")[-1]              # reasoning before the last user turn is cut from history
            parts.append(f"<{m['role']}> {content} <end>")
        text = " ".join(parts) + (" <assistant>" if add_generation_prompt else "")
        return self._ids(text)


CONV = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "two plus two ?"},
        {"role": "assistant", "content": "<think> easy </think> four"}, {"role": "user", "content": "times three ?"},
        {"role": "assistant", "content": "twelve"}]


def test_assistant_spans_by_prefix_rendering():
    tok = WordTokenizer()
    ids, mask, report = render_conversation(tok, CONV)
    words = {v: k for k, v in tok.vocab.items()}
    scored = [[words[i] for i in ids[a:b]] for a, b in completion_spans(mask)]
    assert scored == [["<think>", "easy", "</think>", "four", "<end>"], ["twelve", "<end>"]] and report == {"rewritten": 0, "turns": 2}
    _, last, _ = render_conversation(tok, CONV, last_turn_only=True)
    assert completion_spans(last) == completion_spans(mask)[-1:]
    _, everything, _ = render_conversation(tok, CONV, train_on="all")
    assert everything.all()


def test_history_rewriting_template_is_noticed():
    tok = WordTokenizer(drop_old_reasoning=True)
    ids, mask, report = render_conversation(tok, CONV)
    words = {v: k for k, v in tok.vocab.items()}
    assert report == {"rewritten": 1, "turns": 2}                       # the first turn's tokens changed once it became history
    assert [[words[i] for i in ids[a:b]] for a, b in completion_spans(mask)] == [["twelve", "<end>"]]


def test_corpus_mix_keeps_ratios_on_every_prefix_and_resumes():
    a, b, c = [f"a{i}" for i in range(7)], [f"b{i}" for i in range(50)], [f"c{i}" for i in range(3)]
    mix = CorpusMix([a, b, c], [1, 6, 3], seed=4)
    picks = [next(mix) for _ in range(200)]
    for n in (10, 50, 200):
        counts = np.bincount([i for i, _ in picks[:n]], minlength=3)
        assert np.abs(counts - np.array([0.1, 0.6, 0.3]) * n).max() <= 1.0
    first_epoch_c = [d for i, d in picks if i == 2][:3]
    assert sorted(first_epoch_c) == c                                       # an epoch visits every document once
    resumed = CorpusMix([a, b, c], [1, 6, 3], seed=4)
    for _ in range(120):
        next(resumed)
    state = resumed.state_dict()
    fresh = CorpusMix([a, b, c], [1, 6, 3], seed=4)
    fresh.load_state_dict(state)
    assert [next(fresh) for _ in range(80)] == picks[120:200]
    with pytest.raises(ValueError):
        CorpusMix([a], [0.0])


def test_shards_and_best_fit():
    files = [f"part-{i:03d}.jsonl" for i in range(10)]
    seen = []
    for r in range(4):
        mine, (off, stride) = shard_for_rank(files, r, 4)
        assert (off, stride) == (0, 1)
        seen += mine
    assert sorted(seen) == files
    assert shard_for_rank(files[:2], 3, 4) == (files[:2], (3, 4))
    rng = np.random.default_rng(0)
    lengths = rng.integers(50, 900, size=400).tolist()
    rows = best_fit_rows(lengths, 1024, window=128)
    assert sorted(i for r in rows for i in r) == list(range(400))
    assert all(sum(lengths[i] for i in r) <= 1024 for r in rows)
    sequential, used = 1, 0
    for n in lengths:
        if used + n > 1024:
            sequential, used = sequential + 1, 0
        used += n
    assert len(rows) < 0.93 * sequential                                   # fuller rows than greedy in order


def _identity_worker(rank, world, same):
    from halo_b200.data.packing import pack_documents

    rows = [pack_documents([np.arange(10) + (0 if same else rank)])]
    if same:
        assert_replicas_identical(rows)
    else:
        with pytest.raises(RuntimeError, match="different data"):
            assert_replicas_identical(rows)


@pytest.mark.parametrize("same", [True, False])
def test_replica_identity_is_agreed_on_every_rank(same):
    run_gloo_ranks(_identity_worker, 2, args=(same,), timeout=60.0)
    from halo_b200.data.packing import pack_documents

    assert data_digest([pack_documents([np.arange(5)])]) != data_digest([pack_documents([np.arange(6)])])


def test_bundled_chat_template_extends_history_and_marks_assistant_turns():
    transformers = pytest.importorskip("transformers")
    from tokenizers import Tokenizer, models, pre_tokenizers

    from halo_b200.data.chat_render import load_chat_template, template_ids

    vocab = {chr(i): i - 32 for i in range(32, 127)}
    vocab["\n"], vocab["[UNK]"] = len(vocab), len(vocab) + 1
    tok = Tokenizer(models.WordLevel(vocab, unk_token="[UNK]"))
    tok.pre_tokenizer = pre_tokenizers.Split("", "isolated")
    t = transformers.PreTrainedTokenizerFast(tokenizer_object=tok)
    t.chat_template = load_chat_template()
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}, {"role": "assistant", "content": "hello"},
            {"role": "tool", "content": "42"}, {"role": "assistant", "content": "ok"}]
    ids, mask, report = render_conversation(t, msgs)
    assert report == {"rewritten": 0, "turns": 2}
    texts = [t.decode(ids[a:b]).replace(" ", "") for a, b in completion_spans(mask)]
    assert texts == ["hello<|im_end|>\n", "ok<|im_end|>\n"]
    shorter = template_ids(t, msgs[:3], False)
    assert list(ids[:len(shorter)]) == shorter                                   # history is never rewritten
    with_tools = t.apply_chat_template(msgs[:2], tokenize=False, tools=[{"type": "function", "function": {"name": "calc"}}])
    assert "<tools>" in with_tools and '"name": "calc"' in with_tools and with_tools.count("<|im_start|>system") == 1
    with pytest.raises(FileNotFoundError):
        load_chat_template("nope")


@pytest.mark.parametrize("name,opening,closing", [("llama3", "<|start_header_id|>assistant<|end_header_id|>\n\n", "<|eot_id|>"),
                                                  ("gemma", "<start_of_turn>model\n", "<end_of_turn>"),
                                                  ("mistral", "[/INST]", "</s>"),
                                                  ("harmony", "<|start|>assistant<|channel|>final<|message|>", "<|end|>")])
def test_family_chat_templates_extend_history_and_mark_assistant_turns(name, opening, closing):
    transformers = pytest.importorskip("transformers")
    from tokenizers import Tokenizer, models, pre_tokenizers

    from halo_b200.data.chat_render import load_chat_template, template_ids

    vocab = {chr(i): i - 32 for i in range(32, 127)}
    vocab["\n"], vocab["[UNK]"] = len(vocab), len(vocab) + 1
    tok = Tokenizer(models.WordLevel(vocab, unk_token="[UNK]"))
    tok.pre_tokenizer = pre_tokenizers.Split("", "isolated")
    t = transformers.PreTrainedTokenizerFast(tokenizer_object=tok)
    t.chat_template = load_chat_template(name)
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}, {"role": "assistant", "content": "hello"},
            {"role": "user", "content": "more"}, {"role": "assistant", "content": "ok"}]
    text = t.apply_chat_template(msgs, tokenize=False)
    assert text.count(opening) == 2 and "be brief" in text and text.index("be brief") < text.index("hi")
    ids, mask, report = render_conversation(t, msgs)
    spans = [t.decode(ids[a:b]).replace(" ", "") for a, b in completion_spans(mask)]
    if name != "harmony":
        assert report == {"rewritten": 0, "turns": 2}
        assert spans[0].startswith("hello" + closing.replace(" ", "")) and spans[1].startswith("ok")
        shorter = template_ids(t, msgs[:3], False)
        assert list(ids[:len(shorter)]) == shorter
    else:
        # harmony closes the LAST answer with <|return|> and earlier ones with <|end|>: the earlier turn is a rewrite of
        # what the model saw when it produced it, which the renderer reports instead of hiding
        assert text.endswith("ok<|return|>") and "hello<|end|>" in text and report["rewritten"] == 1
        assert spans[-1].endswith("ok<|return|>")
    prompt = t.apply_chat_template(msgs[:2], tokenize=False, add_generation_prompt=True)
    assert prompt.endswith({"llama3": opening, "gemma": opening, "mistral": "[/INST]", "harmony": "<|start|>assistant"}[name])


def test_near_duplicate_removal(tmp_path):
    """Copies that differ in casing, spacing or a word go; unrelated rows stay; the blocked search equals the one-by-one
    greedy pass whatever the block size; the tool keeps the input order."""
    import json

    from halo_b200.data import deduplication as dd

    rng = np.random.default_rng(0)
    words = ["alpha", "bravo", "charlie", "delta", "echo", "foxtrot", "golf", "hotel", "india", "juliet", "kilo", "lima"]
    base = [" ".join(rng.choice(words, size=30)) for _ in range(40)]
    noisy = [b.upper().replace(" ", "  ") for b in base[:10]] + [b + " mike" for b in base[10:20]]
    texts = base + noisy
    keep = dd.deduplicate_texts(texts, 0.9)
    pairs = [(i, 40 + i) for i in range(20)]
    assert all(keep[a] != keep[b] for a, b in pairs)             # exactly one of each pair survives
    assert keep[20:40].all() and keep.sum() == 40
    v = dd.ngram_vectors(texts)
    for block in (1, 7, 64):
        assert np.array_equal(dd.keep_mask(v, 0.9, block=block), keep)
    in_order = dd.keep_mask(v, 0.9, seed=None)
    assert in_order[:40].all() and not in_order[40:].any()       # unseeded: the first member of a group survives
    src, dst = tmp_path / "in.jsonl", tmp_path / "out.jsonl"
    src.write_text("".join(json.dumps({"id": i, "messages": [{"role": "user", "content": t}]}) + "\n" for i, t in enumerate(texts)))
    assert dd.main([str(src), str(dst), "--field", "messages"]) == 0
    ids = [json.loads(line)["id"] for line in dst.read_text().splitlines()]
    assert ids == sorted(ids) and len(ids) == 40


def test_semantic_vectors_come_from_the_decoder():
    import torch

    from halo_b200.data import deduplication as dd
    from halo_b200.models.config import ModelConfig
    from halo_b200.models.qwen3 import build_model

    class Chars:
        def __call__(self, text, add_special_tokens=False):
            return {"input_ids": [ord(c) % 128 for c in text]}

    cfg = ModelConfig(vocab_size=128, hidden_size=32, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=2, head_dim=16,
                      intermediate_size=64, moe_intermediate_size=0, num_experts=0, model_type="qwen3")
    model = build_model(cfg, device="cpu", seed=0, gradient_checkpointing=False)
    texts = ["the cat sat", "the cat sat", "zzzzqqqq", ""]
    v = dd.model_vectors(texts, model, Chars(), rows_per_pass=3)
    assert v.shape == (4, 32) and torch.allclose(v.norm(dim=1), torch.ones(4), atol=1e-5)
    assert float(v[0] @ v[1]) > 0.9999 and float(v[0] @ v[2]) < 0.9999


def test_tokenizer_pins():
    transformers = pytest.importorskip("transformers")
    from tokenizers import Tokenizer, models

    from halo_b200.entrypoints.script import pin_tokenizer

    tok = Tokenizer(models.WordLevel({"a": 0, "<eos>": 1, "[UNK]": 2}, unk_token="[UNK]"))
    t = transformers.PreTrainedTokenizerFast(tokenizer_object=tok, eos_token="<eos>", padding_side="left")
    assert t.pad_token is None
    pin_tokenizer(t, 4096)
    assert t.pad_token == "<eos>" and t.padding_side == "right" and t.truncation_side == "right" and t.model_max_length == 4096
    t2 = transformers.PreTrainedTokenizerFast(tokenizer_object=tok, eos_token="<eos>", pad_token="a")
    assert pin_tokenizer(t2).pad_token == "a"                  # a shipped pad token is kept
