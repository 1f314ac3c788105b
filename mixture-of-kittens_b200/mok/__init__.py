"""mok: B200-native MoE-layer kernels behind the operator and functional surface of
cursor/mixture-of-kittens (`mok.ops`, `mok.functional`)."""
from . import functional, ops  # noqa: F401
from .functional import MoKConfig, MoKForwardContext, MoKSchedule, MoKWorkspace  # noqa: F401

__all__ = ["functional", "ops", "MoKConfig", "MoKForwardContext", "MoKSchedule", "MoKWorkspace"]
