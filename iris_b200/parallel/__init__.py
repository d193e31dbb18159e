"""Process-level plumbing: control-plane bootstrap, heap mapping helpers, tensor-parallel sharding."""
from .bootstrap import Bootstrap, BootstrapError, SingleBootstrap, TorchDistBootstrap, init_from_env  # noqa: F401
