"""The data-parallel cut of stored rollouts for offline GRPO: whole groups per rank, the same number of rounds on every
rank, an order shared by the ranks of one slice and reshuffled per epoch, and the JSONL source built on it."""

import json

import pytest

from halo_b200.trainers.grpo.group_sampler import GroupSampler


def test_whole_groups_equal_counts_and_a_shared_order():
    ids = [g for g in range(11) for _ in range(4)]                      # 11 groups of 4 rows
    ranks = [GroupSampler(ids, r, 3, groups_per_round=2, seed=5) for r in range(3)]
    assert [len(s) for s in ranks] == [12, 12, 12] and ranks[0].dropped_groups == 2
    seen = set()
    for s in ranks:
        assert s.rounds_per_epoch == 2
        rows = [i for r in range(2) for i in s.round_rows(r)]
        assert s.round_rows(2) is None                                   # one epoch
        for k in range(0, len(rows), 4):                                 # groups arrive whole and consecutive
            assert len({ids[i] for i in rows[k:k + 4]}) == 1
        assert not seen & set(rows)
        seen |= set(rows)
    assert len(seen) == 36
    # the permutation does not depend on the rank (siblings of one slice iterate identical rows) and changes per epoch
    assert ranks[0].order(0) == ranks[2].order(0) and ranks[0].order(0) != ranks[0].order(1)
    twin = GroupSampler(ids, 1, 3, groups_per_round=2, seed=5)
    assert twin.round_rows(1) == ranks[1].round_rows(1)
    two_epochs = [ranks[1].round_rows(r, epochs=2.0) for r in range(5)]
    assert two_epochs[4] is None and sorted(two_epochs[0] + two_epochs[1]) == sorted(two_epochs[2] + two_epochs[3])
    assert two_epochs[0] + two_epochs[1] != two_epochs[2] + two_epochs[3]
    unshuffled = GroupSampler(ids, 0, 1, groups_per_round=11, shuffle=False)
    assert unshuffled.round_rows(0) == list(range(44))
    with pytest.raises(ValueError, match="cannot be cut over 16"):
        GroupSampler(ids, 0, 16)


def test_jsonl_source_cuts_by_rank_and_honours_group_ids(tmp_path):
    from halo_b200.entrypoints.training.grpo import rollouts_from_jsonl

    path = tmp_path / "rollouts.jsonl"
    with open(path, "w") as f:
        for g in range(6):
            for k in range(2):
                # interleaved on disk: the group id, not the position, says which rows belong together
                f.write(json.dumps({"prompt_ids": [g, g], "completion_ids": [k], "reward": float(g + k), "group_id": f"p{g % 6}"}) + "\n")
    sources = [rollouts_from_jsonl(str(path), 2, r, 2, seed=1, prompts_per_round=2) for r in range(2)]
    prompts = []
    for src in sources:
        rounds = [src(0), src(1)]
        assert src(2) is None and all(len(r) == 4 for r in rounds[:1])
        for rnd in rounds:
            for a, b in zip(rnd[::2], rnd[1::2]):
                assert a.prompt_ids.tolist() == b.prompt_ids.tolist()       # both generations of a prompt, together
            prompts += [int(r.prompt_ids[0]) for r in rnd]
    assert sorted(set(prompts)) == list(range(6)) and len(prompts) == 12
