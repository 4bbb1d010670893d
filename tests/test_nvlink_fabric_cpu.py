"""NVLink domain against the fabric the GPUs report: the dump parser, the three pure verdicts, and the collective forms
on gloo ranks fed with stated facts (no GPU, no tool)."""

import pytest

from halo_b200.parallel import nvlink_fabric as F
from tests.common.gloo import run_gloo_ranks

_DUMP = """
==============NVSMI LOG==============
GPU 00000000:1B:00.0
    Product Name                          : NVIDIA B200
    GPU Virtualization Mode
        State                             : None
    Fabric
        State                             : %s
        Status                            : Success
        CliqueId                          : %s
        ClusterUUID                       : 00000000-0000-0000-0000-000000000000
    Processes                             : None
"""


def test_fabric_block_of_the_dump():
    assert F.parse_fabric_clique(_DUMP % ("Completed", "4097")) == 4097
    assert F.parse_fabric_clique(_DUMP % ("Completed", "0")) == F.NO_FABRIC          # a plain 8-GPU baseboard
    assert F.parse_fabric_clique(_DUMP % ("In Progress", "4097")) is None
    assert F.parse_fabric_clique(_DUMP % ("Completed", "N/A")) is None
    assert F.parse_fabric_clique("GPU 0\n    Product Name : X\n") == F.NO_FABRIC      # no Fabric block at all
    # the State of another block is not the fabric's
    assert F.parse_fabric_clique("GPU\n    Other\n        State : Completed\n    Fabric\n        CliqueId : 7\n") is None


def test_verdicts():
    assert F.placement_contradiction(["a"] * 4 + ["b"] * 4, 4) is None
    assert "block(s) [0, 1]" in F.placement_contradiction(["a", "b"] * 4, 4)              # cyclic distribution
    plain = [F.NO_FABRIC] * 16
    assert F.domain_contradiction(plain, [8] * 16, 8, 16) is None
    assert "at most 8" in F.domain_contradiction(plain, [8] * 16, 16, 16)                  # no fabric: a node is the limit
    rack = [11] * 8 + [12] * 8
    assert F.domain_contradiction(rack, [4] * 16, 8, 16) is None
    why = F.domain_contradiction(rack, [4] * 16, 16, 16)
    assert "more than one fabric clique" in why and "{11: 8, 12: 8}" in why
    assert F.narrower_than_fabric([11] * 16, [4] * 16, 4) == 16 and F.narrower_than_fabric([11] * 16, [4] * 16, 16) is None
    assert F.narrower_than_fabric(plain, [8] * 16, 4) is None
    assert "IMEX" in F.mnnvl_prerequisite_reason(False, 5)
    assert "not completed" in F.mnnvl_prerequisite_reason(True, None)
    assert "no fabric clique" in F.mnnvl_prerequisite_reason(True, F.NO_FABRIC)
    assert F.mnnvl_prerequisite_reason(True, 5) is None
    assert not F.imex_channels_present("/nonexistent-directory")


def test_requested_domain_size(monkeypatch):
    monkeypatch.delenv("NVLINK_DOMAIN_SIZE", raising=False)
    assert F.requested_domain_size() is None
    monkeypatch.setenv("NVLINK_DOMAIN_SIZE", "72")
    assert F.requested_domain_size() == 72
    monkeypatch.setenv("NVLINK_DOMAIN_SIZE", "0")
    assert F.requested_domain_size() is None


def _worker(rank: int, world: int):
    host = f"node{rank // 2}"
    # two machines of two GPUs on one fabric clique: a domain of 4 is what the fabric offers
    F.validate_domain(4, world, 2, facts=(21, 2, host))
    F.validate_domain(2, world, 2, facts=(21, 2, host))                                   # narrower: advice only
    with pytest.raises(ValueError, match="more than one fabric clique"):
        F.validate_domain(4, world, 2, facts=(21 + rank // 2, 2, host))
    with pytest.raises(ValueError, match="no GPU reports an NVLink fabric"):
        F.validate_domain(4, world, 2, facts=(F.NO_FABRIC, 2, host))
    with pytest.raises(ValueError, match="not placed 2 to a machine"):
        F.validate_domain(2, world, 2, facts=(21, 2, f"node{rank % 2}"))
    F.validate_domain(4, world, 2, facts=(None if rank == 3 else 21 + rank, 2, host))     # a partial view is no evidence
    # multi-node NVLink prerequisites: refused on every rank when one rank lacks them
    from halo_b200.runtime.consensus import RankFailure

    F.verify_mnnvl_prerequisites(4, 2, facts=(True, 21))
    with pytest.raises(RankFailure, match="rank 2: no IMEX channels"):
        F.verify_mnnvl_prerequisites(4, 2, facts=(rank != 2, 21))
    F.verify_mnnvl_prerequisites(2, 2, facts=(False, None))                                # within a node: nothing to require


def test_collective_checks_on_four_ranks():
    run_gloo_ranks(_worker, 4, timeout=240)
