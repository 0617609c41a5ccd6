"""B200-native Newton constraint solver for InstantMimic's MuJoCo-Warp step.

The package holds the host side of one hot path: ``solve_with_scratch`` and the
M-side factor/solve helpers it shares with the integrator.  All computation is
hand-written CUDA for sm_100a in ``libimnewton.so`` behind the C ABI declared in
``include/imnewton.h``.
"""

from .mjw_step_optimized import (  # noqa: F401
    OptimizedFwdPositionScratch,
    SolverContext,
    make_optimized_fwd_position_scratch,
    solve_with_scratch,
)

__all__ = [
    "OptimizedFwdPositionScratch",
    "SolverContext",
    "make_optimized_fwd_position_scratch",
    "solve_with_scratch",
]
