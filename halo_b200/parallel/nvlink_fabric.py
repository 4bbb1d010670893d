"""Does the declared NVLink domain match the NVLink fabric the GPUs report? Host-side probes only: they read
``nvidia-smi -q`` and a device directory, build no process group and change no setting.

``NVLINK_DOMAIN_SIZE`` says how many consecutive ranks share one NVLink domain (a node's 8 GPUs by default, 72 on an
NVL72 rack). Every "node-local" expert- / context- / tensor-parallel group is a contiguous rank block inside a domain
and moves its data through peer memory, so a domain that is declared wider than the fabric really is would send those
groups over the network while the layout still calls them local. Three checks, each a pure function of gathered facts
plus one collective that gathers them:

* placement: consecutive ranks sit ``gpus_per_node`` to a machine (a cyclic rank distribution breaks the blocks);
* fabric: a domain spans one fabric clique only, and no domain is wider than a node where no fabric exists;
* multi-node NVLink prerequisites when the domain is wider than a node: IMEX channels on every node and a completed
  fabric registration on every GPU, refused by name at start-up rather than as a peer-memory fault in the first dispatch.

The clique is read out of process (``nvidia-smi -q -i <bus id>``): the NVML fabric getters take a versioned struct and a
layout mismatch would take the process down. (The role of halo/distributed/nvlink.py:27-274.)"""

from __future__ import annotations

import functools
import logging
import os
import socket
import subprocess

from halo_b200 import env

log = logging.getLogger(__name__)

NO_FABRIC = -1                      # a definite "this GPU is on no multi-node fabric", unlike None (could not tell)
IMEX_DIR = "/dev/nvidia-caps-imex-channels"


def requested_domain_size() -> int | None:
    """``NVLINK_DOMAIN_SIZE`` as a positive GPU count, or None (unset, or not positive: warned and ignored)."""
    v = env.env_int("NVLINK_DOMAIN_SIZE", None)
    if v is not None and v < 1:
        log.warning("NVLINK_DOMAIN_SIZE=%d is not a positive GPU count: ignored, the domain is one node", v)
        return None
    return v


def parse_fabric_clique(dump: str) -> int | None:
    """The clique id in the ``Fabric`` block of an ``nvidia-smi -q`` dump: an id; NO_FABRIC when the dump has no such
    block or the id is 0 (plain 8-GPU baseboards); None when the registration is not ``Completed`` or the block cannot
    be read. Only the ``Fabric`` block is read - ``State`` occurs elsewhere in the dump."""
    indent = state = clique = None
    for line in dump.splitlines():
        body = line.strip()
        depth = len(line) - len(line.lstrip())
        if indent is None:
            if body == "Fabric":
                indent = depth
            continue
        if body and depth <= indent:
            break
        key, _, value = body.partition(":")
        if key.strip() == "State":
            state = value.strip()
        elif key.strip() == "CliqueId":
            clique = value.strip()
    if indent is None:
        return NO_FABRIC
    if state is None or state.lower() != "completed":
        return None
    try:
        return int(clique) or NO_FABRIC
    except (TypeError, ValueError):
        return None


@functools.lru_cache(maxsize=None)
def _clique_of_bus_id(bus_id: str) -> int | None:
    try:
        out = subprocess.run(["nvidia-smi", "-q", "-i", bus_id], capture_output=True, text=True, timeout=30, check=True)
    except Exception:  # noqa: BLE001 - advisory: a missing tool or a slow driver must not stop start-up
        return None
    return parse_fabric_clique(out.stdout)


def fabric_clique_id(device_index: int | None = None) -> int | None:
    """This process's GPU's fabric clique (cached per device), NO_FABRIC, or None when it cannot be read."""
    try:
        import torch

        if not torch.cuda.is_available():
            return None
        props = torch.cuda.get_device_properties(torch.cuda.current_device() if device_index is None else device_index)
        # by PCI bus id: the tool lists every GPU of the host, the device index counts the visible ones only
        return _clique_of_bus_id(f"{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0")
    except Exception:  # noqa: BLE001
        return None


def placement_contradiction(hosts: list[str], gpus_per_node: int) -> str | None:
    """Why the ranks are not laid out ``gpus_per_node`` to a machine (``hosts[rank]`` = that rank's machine), or None."""
    if gpus_per_node <= 0 or not hosts:
        return None
    bad = {}
    for block in range(len(hosts) // gpus_per_node):
        names = sorted(set(hosts[block * gpus_per_node:(block + 1) * gpus_per_node]))
        if len(names) > 1:
            bad[block] = names
    if not bad:
        return None
    first = min(bad)
    return (f"ranks are not placed {gpus_per_node} to a machine: rank block(s) {sorted(bad)} span more than one machine "
            f"(block {first}: {bad[first]}). Node-local groups are contiguous rank blocks and would reach across machines "
            "through peer memory that does not exist there. Launch one launcher per node with its node rank, or "
            "distribute ranks in blocks, so that consecutive ranks share a machine")


def domain_contradiction(cliques: list[int], node_widths: list[int], domain: int, world: int) -> str | None:
    """Why a declared domain of ``domain`` ranks contradicts the per-rank cliques and node widths, or None. The width
    verdict comes first: ranks without a fabric share one sentinel, so a domain across two such nodes would pass the
    one-clique test."""
    too_wide = {}
    for d, start in enumerate(range(0, world, domain)):
        block = slice(start, start + domain)
        if all(c == NO_FABRIC for c in cliques[block]):
            width = min(node_widths[block])
            if 0 < width < domain:
                too_wide[d] = width
    if too_wide:
        return (f"NVLINK_DOMAIN_SIZE={domain} is wider than a node in domain(s) {sorted(too_wide)}, where no GPU reports an "
                f"NVLink fabric: there is no NVLink between those nodes for a domain to span. Unset it, or set it to at most "
                f"{min(too_wide.values())}")
    split = [d for d in range(world // domain) if len(set(cliques[d * domain:(d + 1) * domain])) > 1]
    if not split:
        return None
    per_clique = {c: cliques.count(c) for c in sorted(set(cliques))}
    return (f"NVLINK_DOMAIN_SIZE={domain} does not match the NVLink fabric: domain(s) {split} span more than one fabric "
            f"clique, so their node-local groups would be part NVLink, part network. Use a size that divides the clique "
            f"size (ranks of this job per clique: {per_clique})")


def narrower_than_fabric(cliques: list[int], node_widths: list[int], domain: int) -> int | None:
    """The NVLink width the job really has on its narrowest node when that exceeds the declared domain (advice: the
    layout could use wider node-local groups), else None."""
    if all(c == NO_FABRIC for c in cliques):
        return None
    widths = [cliques.count(c) for c in set(cliques) - {NO_FABRIC}]
    plain = [w for c, w in zip(cliques, node_widths) if c == NO_FABRIC]
    if plain:
        widths.append(min(plain))
    narrowest = min(widths)
    return narrowest if narrowest > domain else None


def validate_domain(domain: int, world: int, gpus_per_node: int, group=None, facts=None) -> None:
    """COLLECTIVE. Gather (clique, gpus per node, host name) from every rank and refuse a domain the facts contradict;
    every rank decides from the same list, so nobody raises alone. A clique that could not be read anywhere turns the
    fabric checks off (a partial view is no evidence). ``facts`` replaces this rank's own probe (tests)."""
    import torch.distributed as dist

    from halo_b200.runtime.collectives import all_gather_object

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) != world or world <= 1:
        return
    mine = facts if facts is not None else (fabric_clique_id(), gpus_per_node, socket.gethostname())
    every = all_gather_object(tuple(mine), group)
    why = placement_contradiction([e[2] for e in every], gpus_per_node)
    if why:
        raise ValueError(why)
    cliques = [e[0] for e in every]
    if any(c is None for c in cliques):
        return
    widths = [e[1] for e in every]
    why = domain_contradiction(cliques, widths, domain, world)
    if why:
        raise ValueError(why)
    wider = narrower_than_fabric(cliques, widths, domain)
    if wider and dist.get_rank() == 0:
        log.warning("NVLINK_DOMAIN_SIZE=%d is smaller than the NVLink width this job has (%d GPUs share a domain on its "
                    "narrowest node): node-local groups are capped below the fabric", domain, wider)


def imex_channels_present(directory: str = IMEX_DIR) -> bool:
    try:
        return bool(os.listdir(directory))
    except OSError:
        return False


def mnnvl_prerequisite_reason(imex_ok: bool, clique: int | None) -> str | None:
    """Why this rank cannot take part in multi-node NVLink, or None. Asked only where the layout needs it, where an
    unreadable clique means an unfinished fabric registration."""
    if not imex_ok:
        return (f"no IMEX channels in {IMEX_DIR}: peer memory across OS nodes needs the fabric manager and the IMEX "
                "service with matching channels on every node")
    if clique is None:
        return "the GPU's fabric registration is not completed (Fabric State in nvidia-smi -q), or the tool could not be read"
    if clique == NO_FABRIC:
        return "the GPU reports no fabric clique: it is not on a multi-node NVLink fabric"
    return None


def verify_mnnvl_prerequisites(domain: int, gpus_per_node: int, group=None, facts=None) -> None:
    """COLLECTIVE when ``domain > gpus_per_node`` (node-local groups span OS nodes over NVLink): every rank reports its
    IMEX channels and fabric registration and the job refuses by name if any rank lacks them. Otherwise advice only: a
    fabric is present but the domain was never declared. ``facts = (imex_ok, clique)`` replaces the probe (tests)."""
    from halo_b200.runtime import ranks
    from halo_b200.runtime.consensus import reject_across_ranks

    imex_ok, clique = facts if facts is not None else (imex_channels_present(), fabric_clique_id())
    if domain <= gpus_per_node:
        if ranks.is_global_main_process() and requested_domain_size() is None and clique not in (None, NO_FABRIC):
            log.warning("an NVLink fabric is present but NVLINK_DOMAIN_SIZE is unset: node-local groups are capped at %d "
                        "GPUs; declare the domain (72 on an NVL72 rack) to use the fabric", gpus_per_node)
        return
    reason = mnnvl_prerequisite_reason(imex_ok, clique)
    what = f"multi-node NVLink (NVLINK_DOMAIN_SIZE={domain} > gpus_per_node={gpus_per_node})"
    if not ranks.is_distributed():
        if reason:
            log.warning("%s: %s", what, reason)
        return
    reject_across_ranks(reason, group, what)
