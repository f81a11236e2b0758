"""Import-path shim for `from linrec.impl.cuda import ops` (see linrec_b200.ops)."""
from linrec_b200.ops import *  # noqa: F401,F403
from linrec_b200.ops import (  # noqa: F401
    _C, linrec_pipe_bwd, linrec_pipe_fwd, linrec_ref_bwd, linrec_ref_fwd, linrec_tile_bwd, linrec_tile_fwd,
)
