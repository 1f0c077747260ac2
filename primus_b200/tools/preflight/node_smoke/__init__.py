"""Node smoke test: collectors (read-only inventory of one node), per-GPU test tiers run in child processes, an
orchestrator with time limits and an aggregator that turns per-node JSON dumps into a cluster summary.
(Structure of primus/tools/preflight/node_smoke/{collectors,per_gpu,orchestrator,aggregator} in the reference.)"""
from .aggregator import summarize_cluster, write_report  # noqa: F401
from .collectors import collect_all  # noqa: F401
from .orchestrator import run_node_smoke  # noqa: F401
