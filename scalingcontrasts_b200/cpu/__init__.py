"""CPU paths: the float64 oracle and the float32 streamed loss that gloo ranks and in-process simulation use."""
from .oracle import OracleResult, oracle, oracle_loops, relative_l2  # noqa: F401
from .streamed import CpuStreamedLoss, prefix_inverse_norms, simulate_world  # noqa: F401
