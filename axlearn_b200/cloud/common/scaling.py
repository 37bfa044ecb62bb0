"""Aggregates over the scaling specs of an elastic job (reference: axlearn/cloud/common/scaling.py)."""

from __future__ import annotations

from typing import Sequence

from axlearn_b200.cloud.common.job_types import ScalingSpec, Topology


def aggregate_min_resources(scaling_specs: Sequence[ScalingSpec]) -> dict:
    """``min_replicas x resources_per_replica`` summed over the specs: what the job needs to start."""
    totals: dict = {}
    for spec in scaling_specs:
        for resource, count in spec.resources_per_replica.items():
            totals[resource] = totals.get(resource, 0) + count * spec.min_replicas
    return totals


def aggregate_topology(scaling_specs: Sequence[ScalingSpec]) -> list:
    """One ``Topology(topology_per_replica, min_replicas)`` per spec that names a topology."""
    return [Topology(topology=spec.topology_per_replica, replicas=spec.min_replicas)
            for spec in scaling_specs if spec.topology_per_replica]
