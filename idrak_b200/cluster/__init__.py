"""Cluster-level pieces: in-process simulator with failure models and replay, step headers and stop agreement,
control-file steering, topology files, settings advice, link benchmarks."""
from .control import (ClusterRunStopped, ControlFileSteering, HeaderMismatch, StepHeader, StopAgreement, shapes_hash)
from .sim import (ClusterReplay, EventLog, Fault, FaultInjector, InProcessCluster, LinkModel, RankContext, RankDropped,
                  RankTimeout)
from .topology import Topology, advise, load_topology, parse_topology

__all__ = ["ClusterRunStopped", "ControlFileSteering", "HeaderMismatch", "StepHeader", "StopAgreement", "shapes_hash",
           "ClusterReplay", "EventLog", "Fault", "FaultInjector", "InProcessCluster", "LinkModel", "RankContext",
           "RankDropped", "RankTimeout", "Topology", "advise", "load_topology", "parse_topology"]
