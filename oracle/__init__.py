"""CPU oracle for the entmax / lazy attention hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module:
only the test-suite, the smoke entry and the benchmark's CPU-baseline leg do,
and there only as the checker / the timed CPU baseline.

Parity status
-------------
* lazy attention (``lazy_ref``): PINNED.  The dense restatement is checked
  against outputs of the reference's own kernels (``lazy_attention_triton.py``
  executed on CPU through the Triton interpreter); those outputs are stored as
  fixtures under ``tests/golden`` by ``tests/golden/make_lazy_golden.py``.
* alpha-entmax (``entmax_ref``): PARITY UNPINNED beyond analytic known answers.
  The reference checkout does not contain the entmax kernels and its tests
  compare against the third-party ``entmax`` package (``entmax_bisect``,
  unpinned in ``requirements-dev.txt:5``), which is not available offline.
  The mapping is restated from its published definition (unique threshold of
  ``sum_j [x_j - tau]_+^(1/(alpha-1)) = 1``) and pinned only by the known-answer
  cases the reference's tests contain (uniform rows, one-hot rows, padded rows,
  rows summing to one).
"""
from .entmax_ref import (  # noqa: F401
    entmax_ref,
    entmax_bwd_ref,
    entmax_attention_ref,
    entmax_attention_bwd_ref,
    entmax_attention_probs_ref,
    block_mask_ref,
    bisect10_entmax,
    cpu_reference_fwd_bwd,
    entmax_attention_rows_ref,
)
from .lazy_ref import (lazy_attention_ref, lazy_attention_grads_ref,  # noqa: F401
                       lazy_attention_grads_analytic, lazy_attention_rows_ref)
