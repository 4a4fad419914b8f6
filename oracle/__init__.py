"""CPU oracle for the HTile hot path (attention prefill, split-K decode, Mamba-1 scan, Mamba-2 SSD).

THIS PACKAGE IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It restates, on CPU tensors in fp32, the
operators that the CUDA kernel library computes, so that the kernels can be checked.  Only the test
suite, the smoke check and the CPU-baseline / reference legs of the benchmark may import it; the
kernel library and the translator never do, and they raise when the CUDA library is missing rather
than falling back to anything here.

Pinning status
--------------
* ``attention.attention_reference`` (non-causal) restates the reference's own check function
  (tests/test_translators.py:122-135) and ``attention.attention_program`` restates the reference's
  HTile program (tests/data/flash_attention_htile.mlir:40-143).  Both are pinned against outputs of
  the reference's golden Triton translation (tests/golden/flash_attention_triton.py) executed on CPU
  by the Triton interpreter; the stored tiles and the generating script are under ``tests/golden/``.
* Causal masking, bf16, split-K decode, the Mamba-1 selective scan and the Mamba-2 SSD scan do not
  exist in the reference: for them **parity is unpinned** -- the restatements below are the only
  definition, cross-checked only against each other (direct vs. split form, sequential vs. chunked
  form).
"""

from . import attention, decode, inputs, selective_scan, ssd  # noqa: F401
