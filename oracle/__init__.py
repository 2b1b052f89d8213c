"""CPU restatement of the FoldAttention hot paths. TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this directory: it exists so the CUDA
kernels can be checked against an independent statement of the reference's
arithmetic (tests, the smoke check and the benchmark's CPU-baseline leg).

Pinning status
--------------
* `cache_format` (Hadamard butterfly, key/query scales, int8 planes, E4M3
  planes, swizzle, page rows, V sums) is pinned bit-for-bit against outputs of
  the reference's own pure-torch quantisers (`src/fold_attention/decode/cache.py`,
  `src/fold_attention/utils.py`), stored in `tests/golden/cache_format.npz`
  together with the script that generated them.
* `grid` (integer-grid exponents) restates `src/fold_attention/backward/grid.py`,
  which is device-only code: pinned by hand-derived known answers and by the
  bound it documents. Parity with the reference's accumulator *bits* is
  unpinned: those depend on tensor-core accumulation order.
* `backward` is the FP32/FP64 gradient reference of
  `benchmarks/harness/training.py:124-164` and `tests/test_backward.py:79-92`.
* `decode` restates the float64 models the reference's tests hold
  (`tests/test_decode.py:902-928` coarse logit, `:983-1011` mass estimate,
  `:151-153` truncated softmax), pinned against those functions' own outputs
  (`tests/golden/float_models.npz`).
* `tail` restates the decode tail's fit (`src/fold_attention/decode/cache.py:260-337`) and the
  append's block update (`decode/write.py:193-300`); pinned against the reference's `tail_model`
  outputs (`tests/golden/tail_model.npz`) through the effective map, the re-entry points and
  the block rows.
"""
