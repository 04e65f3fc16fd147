"""Python mirror of the C++ GeePsConfig (include/geeps.hpp)."""
from __future__ import annotations

from dataclasses import dataclass, field

DEVICE_CPU, DEVICE_CUDA = 0, 1
TRANSPORT_TCP, TRANSPORT_NVLINK = 0, 1
PARTITION_RANGE, PARTITION_ROUND_ROBIN = 0, 1
TABLE_ADDITIVE, TABLE_SGD_MOMENTUM = 0, 1


@dataclass
class GeePsConfig:
    """Field names and defaults follow the reference's GeePsConfig (include/geeps.hpp:42-71 of the
    reference) for the first thirteen fields; the rest are additions of this framework."""
    num_tables: int = 1
    host_list: list = field(default_factory=lambda: ["127.0.0.1"])
    port_list: list = field(default_factory=list)
    tcp_base_port: int = 9090
    num_comm_channels: int = 1
    output_dir: str = ""
    log_interval: int = 0
    pp_policy: int = 0
    local_opt: int = 1
    gpu_memory_capacity: int = -1          # bytes; -1 = unlimited
    mm_warning_level: int = 1
    pinned_cpu_memory: int = 1
    read_my_writes: int = 0
    # additions
    device: int = DEVICE_CUDA
    cuda_device: int = -1
    transport: int = TRANSPORT_TCP
    partitioner: int = PARTITION_RANGE
    table_mode: int = TABLE_ADDITIVE
    table_modes: dict = field(default_factory=dict)   # table id -> mode
    # table id -> first row that is also published in fp32 (rows below it reach the bf16 caches only)
    table_fp32_from_row: dict = field(default_factory=dict)
    # table id -> 1: uncached ("pull") table of the NVLINK transport: workers keep no copy, reads fetch from the shards
    table_pull: dict = field(default_factory=dict)
    # table id -> the range partition hands out rows in groups of this many
    table_partition_align: dict = field(default_factory=dict)
    learning_rate: float = 0.01
    momentum: float = 0.9
    weight_decay: float = 0.0
    grad_scale: float = 1.0
    bf16_compute_cache: int = 0
    use_multicast: int = 0     # NVLINK transport: reduce / publish through an NVSwitch multicast mapping (multimem)
    device_wait_budget_us: int = 30_000_000
    host_wait_budget_ms: int = 0
    heartbeat_timeout_ms: int = 30000
    snapshot_dir: str = ""
    snapshot_interval: int = 0
    num_workers_override: int = 0

    _NUMERIC = ("num_tables", "tcp_base_port", "num_comm_channels", "log_interval", "pp_policy", "local_opt",
                "gpu_memory_capacity", "mm_warning_level", "pinned_cpu_memory", "read_my_writes", "device",
                "cuda_device", "transport", "partitioner", "table_mode", "learning_rate", "momentum",
                "weight_decay", "grad_scale", "bf16_compute_cache", "use_multicast", "device_wait_budget_us",
                "host_wait_budget_ms", "heartbeat_timeout_ms", "snapshot_interval", "num_workers_override")
    _STRING = ("output_dir", "snapshot_dir")
