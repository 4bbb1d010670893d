"""Environment knobs of the framework, read through one small set of typed readers.

Names keep the reference's prefixes (``HALO_``, ``DIST_``, ``NVLINK_``) so an existing launch
environment carries over (halo/env.py:33-158). A blank value counts as unset; a malformed value
warns once and falls back to the default rather than silently flipping a knob.
"""

from __future__ import annotations

import logging
import os
from datetime import timedelta

log = logging.getLogger(__name__)

_TRUE = frozenset({"1", "true", "yes", "on"})
_FALSE = frozenset({"0", "false", "no", "off"})
_warned: set[str] = set()

DEFAULT_NCCL_TIMEOUT_MINUTES = 30
DEFAULT_STORE_TIMEOUT_HOURS = 4
DEFAULT_FS_PROBE_TIMEOUT_SECONDS = 60
WATCHDOG_WARN_FRACTION = 0.8

# every knob this package reads, with its meaning (kept complete by tests/test_conventions_cpu.py)
CATALOGUE = {
    "HALO_DATA_ROOT": "scratch directory for profiles, caches and run logs",
    "HALO_LOG_LEVEL": "root log level of the framework's handler",
    "HALO_WEIGHT_SYNC_CHUNK_MB": "size of one packed trainer->rollout weight chunk",
    "HALO_WEIGHT_SYNC_GATHER_AHEAD": "expert layers gathered ahead of the one being sent",
    "HALO_EP_CAPACITY_FACTOR": "receive-buffer rows per rank as a multiple of the mean load",
    "HALO_KERNEL_WAIT_MS": "host-side bound on waits for a device event",
    "HALO_BOUNDED_WAIT_SECONDS": "deadline of a bounded stream wait in weight sync",
    "HALO_ROLLOUT_WAIT_SECONDS": "how long a trainer waits for a round from its rollout rank",
    "HALO_GEMM_PAIR": "CTA-pair GEMM: 1 where it wins (default), 0 never, 2 everywhere",
    "HALO_ATTN_BWD_VARIANT": "backward attention kernels (2 = double-buffered score tiles and eight element-wise warps, the default; 1 = the first form)",
    "HALO_ATTN_FWD_VARIANT": "forward attention kernel form (3 = output and probabilities kept in TMEM, the default; 2 = probabilities through shared memory; 1 = 128-key tiles)",
    "HALO_WEIGHT_SYNC_NVLS": "trainer -> rollout weight push through NVLink multicast stores when the arena supports it (default 1)",
    "HALO_ZERO_NVLS": "sharded optimizer: reduce and all-gather through NVLink multicast (multimem) when the buffers support it (default 0: plain peer loads / stores, bit-identical to the unsharded optimizer)",
    "HALO_MOE_FUSED": "expert products with the token movement inside the GEMM kernels (1, default) or as separate push / pull kernels (0)",
    "HALO_CP_DIRECT_READS": "context parallelism: flash kernels read foreign key / value tiles from their owners on every use (1) instead of from a local mirror filled once per exchange (0, default)",
    "HALO_PEER_WAIT_MS": "how long a kernel waits for rows or a flag from a peer GPU before it gives up with a status (default 20000)",
    "HALO_ROW_BLOCKS_PER_SM": "thread blocks per SM of the expert row kernels (dispatch / combine)",
    "HALO_NNODES": "nodes of a multi-node launch (read by the CLI when --nnodes is not given)",
    "HALO_NODE_RANK": "this node's index in a multi-node launch",
    "HALO_RDZV_ENDPOINT": "host:port of the first node, the rendezvous address of a multi-node launch",
    "DIST_NCCL_TIMEOUT_MINUTES": "collective watchdog of every process group",
    "DIST_STORE_TIMEOUT_HOURS": "timeout of store-based joins that outlast the watchdog",
    "DIST_FS_PROBE_TIMEOUT_SECONDS": "how long to poll for the shared-filesystem sentinel",
    "DIST_SHARED_FILESYSTEM": "inputs and outputs are on storage every node sees (default of the two flags below; single-node jobs default to 1)",
    "DIST_INPUT_SHARED_FILESYSTEM": "inputs are on a filesystem every node sees",
    "DIST_OUTPUT_SHARED_FILESYSTEM": "outputs go to a filesystem every node sees",
    "NVLINK_DOMAIN_SIZE": "ranks per NVLink domain (overrides detection)",
}


# knobs that legitimately differ between ranks or nodes of one job; every other catalogued knob must be the same everywhere
PER_RANK = frozenset({"HALO_NODE_RANK", "HALO_DATA_ROOT", "HALO_LOG_LEVEL"})


def rank_uniform_snapshot() -> dict[str, str | None]:
    """The raw values of every catalogued knob that all ranks of a job must agree on (unset: None)."""
    return {name: _raw(name) for name in sorted(CATALOGUE) if name not in PER_RANK}


def _raw(name: str) -> str | None:
    v = os.environ.get(name)
    return v if v is not None and v.strip() else None


def _warn_once(name: str, msg: str) -> None:
    if name not in _warned:
        _warned.add(name)
        log.warning(msg)


def env_flag(name: str, default: bool = False) -> bool:
    v = _raw(name)
    if v is None:
        return default
    low = v.strip().lower()
    if low in _TRUE:
        return True
    if low in _FALSE:
        return False
    _warn_once(name, f"ignoring {name}={v!r}: expected one of 1/true/yes/on/0/false/no/off; using {default}")
    return default


def env_int(name: str, default: int | None) -> int | None:
    v = _raw(name)
    if v is None:
        return default
    try:
        return int(v)
    except ValueError:
        _warn_once(name, f"ignoring {name}={v!r}: expected an integer; using {default}")
        return default


def env_float(name: str, default: float | None) -> float | None:
    v = _raw(name)
    if v is None:
        return default
    try:
        return float(v)
    except ValueError:
        _warn_once(name, f"ignoring {name}={v!r}: expected a number; using {default}")
        return default


def env_positive_int(name: str, default: int) -> int:
    v = env_int(name, default)
    if v is None or v < 1:
        _warn_once(name, f"ignoring {name}={v!r}: expected a positive integer; using {default}")
        return default
    return v


def env_non_negative_int(name: str, default: int) -> int:
    v = env_int(name, default)
    if v is None or v < 0:
        _warn_once(name, f"ignoring {name}={v!r}: expected a non-negative integer; using {default}")
        return default
    return v


def env_positive_float(name: str, default: float) -> float:
    v = env_float(name, default)
    if v is None or v <= 0:
        _warn_once(name, f"ignoring {name}={v!r}: expected a positive number; using {default}")
        return default
    return v


def env_str(name: str, default: str | None = None) -> str | None:
    v = os.environ.get(name)
    return default if v is None else v


def nccl_timeout() -> timedelta:
    return timedelta(minutes=env_positive_int("DIST_NCCL_TIMEOUT_MINUTES", DEFAULT_NCCL_TIMEOUT_MINUTES))


def store_timeout() -> timedelta:
    return timedelta(hours=env_positive_int("DIST_STORE_TIMEOUT_HOURS", DEFAULT_STORE_TIMEOUT_HOURS))


def fs_probe_timeout() -> timedelta:
    return timedelta(seconds=env_positive_int("DIST_FS_PROBE_TIMEOUT_SECONDS", DEFAULT_FS_PROBE_TIMEOUT_SECONDS))


def watchdog_bounded_seconds() -> float:
    """Longest one rank may block outside a collective before its peers' watchdog is at risk."""
    return nccl_timeout().total_seconds() * WATCHDOG_WARN_FRACTION


def data_root() -> str:
    return env_str("HALO_DATA_ROOT") or os.path.join(os.path.expanduser("~"), ".cache", "halo_b200")


def data_path(*parts: str) -> str:
    return os.path.join(data_root(), *parts)


def torch_trace_dir() -> str:
    return data_path("profiling", "torch")


def weight_sync_chunk_bytes() -> int:
    return env_positive_int("HALO_WEIGHT_SYNC_CHUNK_MB", 1024) * 1024 * 1024


def weight_sync_gather_ahead() -> int:
    return env_non_negative_int("HALO_WEIGHT_SYNC_GATHER_AHEAD", 1)


def weight_sync_nvls() -> bool:
    return env_flag("HALO_WEIGHT_SYNC_NVLS", True)


def zero_nvls() -> bool:
    return env_flag("HALO_ZERO_NVLS", False)


def cp_direct_reads() -> bool:
    return env_flag("HALO_CP_DIRECT_READS", False)


def moe_fused() -> bool:
    return env_flag("HALO_MOE_FUSED", True)


def ep_capacity_factor() -> float:
    return env_positive_float("HALO_EP_CAPACITY_FACTOR", 1.5)
