"""Tool protocols, the tool environment and environment-driven rollouts on CPU: ReAct and tagged tool calls parse and
refuse malformed turns, a scripted policy solves a tool task through the episode loop, and episodes played by the
job's own sampler become training rows whose masks mark exactly the sampled tokens."""

import asyncio

import numpy as np
import pytest
import torch

from halo_b200.environments.base import Turn
from halo_b200.environments.episode_loop import play_episode
from halo_b200.environments.protocols import MalformedTurn, ToolCall, calculator, default_tools, parse_native, parse_react
from halo_b200.environments.registry import environment_types, make_environment


def test_protocol_parsers():
    t = parse_native(Turn("assistant", 'I will compute. <tool_call>{"name": "calculator", "arguments": {"expression": "2+2"}}</tool_call>'))
    assert t.calls == [ToolCall("calculator", {"expression": "2+2"}, "call_0")] and t.final_answer is None
    assert parse_native(Turn("assistant", "The answer is 4.")).final_answer == "The answer is 4."
    structured = Turn("assistant", "", tool_calls=[{"id": "x1", "function": {"name": "calculator", "arguments": '{"expression": "1"}'}}])
    assert parse_native(structured).calls[0].call_id == "x1"
    for bad in ('<tool_call>{"name": "calculator", </tool_call>', "<tool_call>{}</tool_call>", "<tool_call> never closed"):
        with pytest.raises(MalformedTurn):
            parse_native(Turn("assistant", bad))
    r = parse_react(Turn("assistant", 'Thought: add them\nAction: calculator\nAction Input: {"expression": "3*7"}\nObservation: 22'))
    assert r.calls[0].name == "calculator" and r.calls[0].arguments == {"expression": "3*7"} and r.thought == "add them"
    assert parse_react(Turn("assistant", "Thought: done\nFinal Answer: 21")).final_answer == "21"
    assert parse_react(Turn("assistant", "Action: search\nAction Input: capital of France")).calls[0].arguments == {"input": "capital of France"}
    with pytest.raises(MalformedTurn, match="neither"):
        parse_react(Turn("assistant", "I think it is 21"))


def test_tools_check_arguments_and_never_execute_code():
    reg = default_tools()
    assert reg.call(ToolCall("calculator", {"expression": "(3 + 4) * 2 ** 3"})) == "56"
    assert "missing ['expression']" in reg.call(ToolCall("calculator", {}))
    assert "unknown ['x']" in reg.call(ToolCall("calculator", {"expression": "1", "x": 2}))
    assert reg.call(ToolCall("shell", {})).startswith("error: no tool named")
    assert reg.call(ToolCall("calculator", {"expression": "__import__('os').getcwd()"})).startswith("error:")
    assert calculator("7 // 2") == "3"
    assert reg.definitions()[0]["function"]["parameters"]["required"] == ["expression"]


@pytest.mark.parametrize("protocol", ["native", "react"])
def test_scripted_policy_solves_a_tool_task(protocol):
    assert "tool_qa" in environment_types()
    script = {
        "native": ['<tool_call>{"name": "calculator", "arguments": {"expression": "17*23"}}</tool_call>', "It is \\boxed{391}"],
        "react": ["no format at all", 'Thought: multiply\nAction: calculator\nAction Input: {"expression": "17*23"}', "Final Answer: 391"],
    }[protocol]
    seen = []

    async def policy(messages, tools):
        seen.append((messages[-1], tools))
        return Turn("assistant", script[len(seen) - 1])

    env = make_environment("tool_qa", {"question": "What is 17 x 23?", "answer": "391"}, protocol=protocol)
    rec = asyncio.run(play_episode(env, policy))
    assert rec.score == 1.0 and rec.done_reason == "answered" and rec.tool_calls_used == 1
    observation = seen[-1][0]
    assert "391" in observation["content"] and observation["role"] == ("tool" if protocol == "native" else "user")
    if protocol == "native":
        assert seen[0][1][0]["function"]["name"] == "calculator"
    else:
        assert "could not be used" in seen[1][0]["content"]            # the malformed first turn was answered with a correction


class ByteTokenizer:
    """Code points 0..263 are tokens (text round-trips exactly, whatever a random policy samples); 256..259 also mark
    the roles and 260 ends a turn. Rendering a longer conversation extends the rendering of a shorter one, as chat
    templates that do not rewrite history do."""

    eos_token_id = 260
    ROLES = {"system": 256, "user": 257, "assistant": 258, "tool": 259}

    def apply_chat_template(self, messages, add_generation_prompt=True, tokenize=True, tools=None):
        ids = []
        for m in messages:
            ids += [self.ROLES[m["role"]]] + [ord(c) for c in m["content"]] + [self.eos_token_id]
        return ids + ([self.ROLES["assistant"]] if add_generation_prompt else [])

    def decode(self, ids, skip_special_tokens=False):
        return "".join(chr(i) for i in ids if i != self.eos_token_id)


def test_sampled_episodes_become_masked_rows():
    from halo_b200.inference.generate import SamplingParams
    from halo_b200.models.config import ModelConfig
    from halo_b200.models.qwen3 import build_model
    from halo_b200.trainers.grpo.environment_rollouts import EnvironmentRolloutSource
    from halo_b200.trainers.grpo.trainer import build_grpo_batch

    cfg = ModelConfig(vocab_size=264, hidden_size=32, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
                      head_dim=16, intermediate_size=64, moe_intermediate_size=0, num_experts=0, model_type="qwen3")
    model = build_model(cfg, device="cpu", seed=0, gradient_checkpointing=False)
    tasks = [{"question": "What is 2 + 2?", "answer": "4"}, {"question": "What is 3 * 3?", "answer": "9"}]
    src = EnvironmentRolloutSource(model, ByteTokenizer(), tasks, "tool_qa", num_generations=2,
                                   sampling=SamplingParams(max_new_tokens=6), tasks_per_round=2,
                                   env_options={"protocol": "react"}, seed=1)
    rollouts = src(0)
    assert len(rollouts) == 4 and src.drifted == 0
    tok = ByteTokenizer()
    for r, rec in zip(rollouts, src.last_records):
        mask = r.completion_mask
        assert len(mask) == len(r.completion_ids) == len(r.sampler_logprobs)
        # a random policy never follows the format: three turns (two corrections) of up to six sampled tokens each
        assert 3 <= int(mask.sum()) <= 18 and rec.done_reason == "malformed_turns"
        assert (r.sampler_logprobs[mask == 0] == 0).all() and (r.sampler_logprobs[mask == 1] < 0).all()
        # the environment's tokens inside the row are the corrective user turns, rendered by the template
        between = "".join(chr(int(t)) for t, m in zip(r.completion_ids, mask) if m == 0)
        assert between.count("could not be used") == 2
        # the row is what a fresh rendering of the whole conversation gives (up to the last sampled token)
        full = tok.apply_chat_template(rec.messages, add_generation_prompt=False)
        row = np.concatenate([r.prompt_ids, r.completion_ids]).tolist()
        assert full[:len(row)] == row
    batch = build_grpo_batch(rollouts, torch.zeros(4), torch.zeros(4, dtype=torch.bool))
    assert int((batch.labels != -100).sum()) == sum(int(r.completion_mask.sum()) for r in rollouts)
    with torch.no_grad():
        logp, _ = model.token_logprobs(batch.input_ids, batch.position_ids, batch.cu_seqlens, batch.labels)
    scored = batch.labels.reshape(-1) != -100
    assert torch.allclose(logp[scored], batch.old_logprobs[scored], atol=1e-4)       # sampler and trainer agree token by token


def test_environment_evaluation_report():
    from halo_b200.entrypoints.env_eval import evaluate_tasks
    from halo_b200.inference.generate import SamplingParams
    from halo_b200.models.config import ModelConfig
    from halo_b200.models.qwen3 import build_model

    cfg = ModelConfig(vocab_size=264, hidden_size=32, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1,
                      head_dim=16, intermediate_size=64, moe_intermediate_size=0, num_experts=0, model_type="qwen3")
    model = build_model(cfg, device="cpu", seed=0, gradient_checkpointing=False)
    tasks = [{"question": "2 + 2?", "answer": "4"}, {"question": "3 * 3?", "answer": "9"}]
    report, episodes = evaluate_tasks(model, ByteTokenizer(), tasks, "tool_qa", 2, SamplingParams(max_new_tokens=4, seed=None),
                                      {"protocol": "native"})
    # under the tagged-call protocol free text is a final answer: a random policy answers at once, wrongly
    assert report["episodes"] == 4 and report["tasks"] == 2 and report["mean_score"] == 0.0 and report["pass@2"] == 0.0
    assert report["cut_short"] == 0.0 and all(e["done_reason"] == "answered" and e["n_turns"] == 1 and len(e["turns"]) == 1 for e in episodes)
