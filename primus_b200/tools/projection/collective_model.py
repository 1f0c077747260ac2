"""Analytic collective-time model (seconds) for a node with uniform all-to-all links (NVSwitch) and a slower
scale-out fabric between nodes.

Per collective the model returns ``launch + fixed overhead + latency term + bytes term / effective
bandwidth``; collectives that span nodes are split hierarchically (intra-node phase at NVLink bandwidth,
inter-node phase at NIC bandwidth).  Defaults follow the reference's model
(primus/core/projection/module_profilers/collective_args.py:14-110, collective_model.py:392-422,776-881):
bandwidth efficiency 0.70 (0.80 for point-to-point), fixed overhead 200 us for all-reduce / 150 us for
all-to-all, 2.8 us launch, ring all-reduce time ``2 [(p-1) lat + S (p-1)/p / bw]``.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class Hardware:
    name: str = "b200"
    gpus_per_node: int = 8
    hbm_gb: float = 180.0
    hbm_gbs: float = 6551.0
    bf16_tflops: float = 1649.0
    bf16_tflops_sustained: float = 1391.0
    fp8_tflops: float = 3300.0
    node_bw_gbs: float = 770.0      # per direction per GPU inside the node
    node_lat_us: float = 2.0
    pod_bw_gbs: float = 50.0        # per GPU across nodes
    pod_lat_us: float = 5.0
    bw_eff: float = 0.70
    p2p_bw_eff: float = 0.80
    ar_overhead_us: float = 200.0
    a2a_overhead_us: float = 150.0
    launch_us: float = 2.8
    nvls: bool = True

    @classmethod
    def from_yaml(cls, d: dict) -> "Hardware":
        return cls(
            name=d.get("name", "hw"), gpus_per_node=d.get("gpus_per_node", 8), hbm_gb=d.get("hbm_gb", 180),
            hbm_gbs=d.get("hbm_gbs_measured", d.get("hbm_gbs_nominal", 6551)),
            bf16_tflops=d.get("bf16_tflops_measured", d.get("bf16_tflops_nominal", 1649)),
            bf16_tflops_sustained=d.get("bf16_tflops_sustained", d.get("bf16_tflops_measured", 1391)),
            fp8_tflops=d.get("fp8_tflops_nominal", 4500) * 0.73,
            node_bw_gbs=d.get("node_bw_gbs_measured", d.get("node_bw_gbs", 770)), node_lat_us=d.get("node_lat_us", 2.0),
            pod_bw_gbs=d.get("pod_bw_gbs", 50), pod_lat_us=d.get("pod_lat_us", 5.0), bw_eff=d.get("bw_eff", 0.70),
            p2p_bw_eff=d.get("p2p_bw_eff", 0.80), nvls=d.get("nvls", False))


class CollectiveModel:
    def __init__(self, hw: Hardware):
        self.hw = hw

    def _split(self, p: int) -> tuple[int, int]:
        """(ranks inside a node, number of nodes) for a group of p ranks placed densely."""
        g = self.hw.gpus_per_node
        return (p, 1) if p <= g else (g, -(-p // g))

    def _bw(self, inter: bool, p2p: bool = False) -> float:
        raw = self.hw.pod_bw_gbs if inter else self.hw.node_bw_gbs
        return raw * 1e9 * (self.hw.p2p_bw_eff if p2p else self.hw.bw_eff)

    def _lat(self, inter: bool) -> float:
        return (self.hw.pod_lat_us if inter else self.hw.node_lat_us) * 1e-6

    def _ring(self, nbytes: float, p: int, inter: bool, passes: int) -> float:
        if p <= 1:
            return 0.0
        return passes * ((p - 1) * self._lat(inter) + nbytes * (p - 1) / p / self._bw(inter))

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, nbytes: float, p: int) -> float:
        if p <= 1 or nbytes <= 0:
            return 0.0
        hw = self.hw
        local, nodes = self._split(p)
        base = (hw.launch_us + hw.ar_overhead_us) * 1e-6
        if nodes == 1:
            if hw.nvls:  # in-switch reduction: one pass of the data up and one down
                return base + 2 * self._lat(False) + nbytes / self._bw(False) * 1.05
            return base + self._ring(nbytes, local, False, 2)
        # hierarchical: reduce-scatter in the node, all-reduce across nodes on 1/local of the data, all-gather
        t = self._ring(nbytes, local, False, 1) + self._ring(nbytes / local, nodes, True, 2) + self._ring(nbytes, local, False, 1)
        return base + 0.9 * t + 0.1 * t  # phases are pipelined by the library; keep the sum as the estimate

    def reduce_scatter(self, nbytes: float, p: int) -> float:
        """nbytes = size of the full (input) buffer."""
        if p <= 1 or nbytes <= 0:
            return 0.0
        local, nodes = self._split(p)
        base = (self.hw.launch_us + self.hw.ar_overhead_us / 2) * 1e-6
        if nodes == 1:
            return base + self._ring(nbytes, local, False, 1)
        return base + self._ring(nbytes, local, False, 1) + self._ring(nbytes / local, nodes, True, 1)

    def all_gather(self, nbytes: float, p: int) -> float:
        """nbytes = size of the full (output) buffer."""
        return self.reduce_scatter(nbytes, p)

    def all_to_all(self, nbytes: float, p: int) -> float:
        """nbytes = bytes every rank sends in total (to all peers)."""
        if p <= 1 or nbytes <= 0:
            return 0.0
        local, nodes = self._split(p)
        base = (self.hw.launch_us + self.hw.a2a_overhead_us) * 1e-6
        intra_bytes = nbytes * (local - 1) / p
        inter_bytes = nbytes * (p - local) / p
        t = (local - 1) * self._lat(False) * 0.25 + intra_bytes / self._bw(False)
        if nodes > 1:
            t = max(t, (nodes - 1) * self._lat(True) + inter_bytes / self._bw(True))
        return base + t

    def send_recv(self, nbytes: float, inter_node: bool = False) -> float:
        if nbytes <= 0:
            return 0.0
        return self.hw.launch_us * 1e-6 + self._lat(inter_node) + nbytes / self._bw(inter_node, p2p=True)

    def broadcast(self, nbytes: float, p: int) -> float:
        if p <= 1:
            return 0.0
        local, nodes = self._split(p)
        t = self._lat(False) * 2 + nbytes / self._bw(False)
        if nodes > 1:
            t += self._lat(True) * 2 + nbytes / self._bw(True)
        return self.hw.launch_us * 1e-6 + t
