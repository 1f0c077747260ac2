"""Parallel-plan search: enumerate legal plans, keep those that fit in memory, rank by projected throughput."""
