"""CPU checker for the score -> select -> compact path.  TEST INFRASTRUCTURE ONLY.

This package restates, in plain torch-on-CPU / numpy, the arithmetic of the
reference's own PyTorch scoring path, its group selector and its paged
compaction, each function citing the reference file:line it follows.  It is
used by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline leg
of ``bench.py`` as the checker and the timed baseline.  Nothing in the product
package imports it, and it is never a fallback for the CUDA kernels.

Pinning: the reference publishes no tests or golden vectors for this path, so
the restatement is pinned against outputs of the reference itself, produced by
importing the reference in the build container
(``tests/golden/make_golden.py``) and committed as fixtures under
``tests/golden/``; ``tests/test_oracle_golden.py`` replays them.
"""
from .scoring import (  # noqa: F401
    geometric_offsets,
    score_keys_reference,
    score_keys_exact64,
)
from .selection import (  # noqa: F401
    streaming_moments,
    select_group_per_head,
    select_layer_local,
    final_scores_group_per_head,
    topk_lowest_index,
)
from .compaction import (  # noqa: F401
    split_kv_axes,
    gather_request_k_dense,
    compact_per_head,
    compact_shared,
    truncate_tail_blocks,
    fallback_keep_indices,
)
from . import input_patch  # noqa: F401,E402
