"""The tuner's cost model: T = max(T_compute, T_memory) + T_sync + T_launch (src/autotune/cost_model.cpp:32-49,
include/halo/autotune/cost_model.h).  T_memory = bytes / measured bandwidth of the tier the operands live in, scaled by
min(1, parallelism / the thread count the bandwidth was measured with); T_compute = flops / (calibrated GFLOP/s per
worker x workers).  There is no built-in throughput constant: bandwidth comes from measured rows of the profile
database, the per-worker throughput from calibrate_gflops_per_thread on a measured run.  On the cuda backend a "worker"
is one SM and the tier is "vram"."""
from __future__ import annotations

import math
from dataclasses import dataclass, field


@dataclass
class CostInputs:
    """What one candidate does, as reported by its tunable operator."""
    flops: float = 0.0
    bytes: int = 0
    tier: str = "host"
    parallelism: int = 1  # workers that actually get work
    launches: int = 1
    syncs: int = 0


@dataclass
class CostEstimate:
    t_compute_ns: float = 0.0
    t_memory_ns: float = 0.0
    t_sync_ns: float = 0.0
    t_launch_ns: float = 0.0
    total_ns: float = 0.0
    memory_bound: bool = False  # the model's classification (t_memory >= t_compute), not counter-verified

    def to_json(self) -> dict:
        return {"t_compute_ns": self.t_compute_ns, "t_memory_ns": self.t_memory_ns, "t_sync_ns": self.t_sync_ns,
                "t_launch_ns": self.t_launch_ns, "total_ns": self.total_ns, "memory_bound_estimate": self.memory_bound}


@dataclass
class CostModel:
    bandwidth_gbps: dict[str, float] = field(default_factory=dict)  # per tier, GB/s
    bandwidth_threads: int = 1
    gflops_per_thread: float = 0.0
    launch_ns: float = 0.0
    sync_ns: float = 0.0

    @staticmethod
    def from_measurements(measured: list[dict], gflops_per_thread: float, launch_ns: float = 0.0, sync_ns: float = 0.0) -> "CostModel":
        """measured: rows {tier, threads, read_gbps (the MEDIAN of the measured read bandwidth)}; refuses an empty list, a
        non-positive bandwidth and inconsistent thread counts."""
        if not measured:
            raise ValueError("cost model: no tier bandwidth measurements (Config)")
        m = CostModel(gflops_per_thread=gflops_per_thread, launch_ns=launch_ns, sync_ns=sync_ns, bandwidth_threads=int(measured[0]["threads"]))
        for t in measured:
            if int(t["threads"]) != m.bandwidth_threads or m.bandwidth_threads < 1:
                raise ValueError(f"cost model: tier bandwidths measured with different thread counts ({t['threads']} vs {m.bandwidth_threads}) (Config)")
            bw = float(t["read_gbps"])
            if not math.isfinite(bw) or bw <= 0:
                raise ValueError(f"cost model: tier {t['tier']} median read bandwidth {bw} is not positive (Config)")
            m.bandwidth_gbps[str(t["tier"])] = bw
        return m

    def estimate(self, c: CostInputs) -> CostEstimate:
        if not (self.gflops_per_thread > 0 and math.isfinite(self.gflops_per_thread)):
            raise ValueError(f"cost model: gflops_per_thread {self.gflops_per_thread} is not calibrated (Config)")
        bw = self.bandwidth_gbps.get(c.tier, 0.0)
        if not bw > 0:
            raise ValueError(f"cost model: no measured bandwidth for tier {c.tier} (Config)")
        if not (c.flops >= 0 and math.isfinite(c.flops)):
            raise ValueError("cost model: invalid flops (Config)")
        par = max(1, c.parallelism)
        bw_scale = min(1.0, par / max(1, self.bandwidth_threads))
        e = CostEstimate()
        e.t_compute_ns = c.flops / (self.gflops_per_thread * par)  # GFLOP/s == flop/ns
        e.t_memory_ns = c.bytes / (bw * bw_scale)                  # GB/s == B/ns
        e.t_sync_ns = self.sync_ns * c.syncs
        e.t_launch_ns = self.launch_ns * c.launches
        e.total_ns = max(e.t_compute_ns, e.t_memory_ns) + e.t_sync_ns + e.t_launch_ns
        e.memory_bound = e.t_memory_ns >= e.t_compute_ns
        return e


def calibrate_gflops_per_thread(flops: float, measured_ns: float, threads: int) -> float:
    """Per-worker GFLOP/s from one measured run of one of this backend's own kernels: flops / (ns x workers)."""
    if not (flops > 0 and measured_ns > 0 and threads > 0 and math.isfinite(flops) and math.isfinite(measured_ns)):
        raise ValueError("calibrate_gflops_per_thread: invalid inputs (Config)")
    return flops / (measured_ns * threads)
