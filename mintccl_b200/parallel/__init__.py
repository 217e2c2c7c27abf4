"""Communicators, control plane, CPU reference backend and tensor-parallel layers."""
from .rendezvous import ControlPlane, SingleControl, TorchDistControl, MpiControl, connect  # noqa: F401
