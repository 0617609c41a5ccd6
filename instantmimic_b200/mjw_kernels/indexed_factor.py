"""placeholder"""
def create_blocked_dense_factor_solve_scratch(m, d, device=None, **kw):
    return None
