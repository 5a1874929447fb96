"""CPU oracle for the attention hot path (TEST INFRASTRUCTURE, not product code).

Everything under ``oracle/`` is a CPU restatement of the reference's algorithms
for paged-attention decode, FP8-e4m3 KV quantisation, chunked prefill and
RMSNorm.  It exists so the CUDA kernels can be checked against it.  Only the
test-suite, the smoke check and the CPU-baseline leg of the benchmark may import
it; the shipped package never does and fails loudly without its CUDA library.

Parity status: pinned.  ``tests/golden/*.npz`` were produced by importing the
reference's own Python modules (``tests/golden/make_golden.py`` is the
generating script) and ``tests/test_oracle_golden.py`` checks every function of
this package against those vectors, which include the set-ups of the reference's
own known-answer tests.
"""
