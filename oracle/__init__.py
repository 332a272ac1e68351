"""CPU oracle for the packed-matvec path.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Everything in this package is a numpy restatement of the arithmetic that
mlkit (the reference library) performs for its packed-inference path:

* ``bitstream``   little-endian unsigned bit streams (pack / unpack)
* ``codec``       grouped scalar decode, round-to-nearest encode
* ``transforms``  Walsh-Hadamard, Paley / DCT factor bases, structured and
                  randomized transforms
* ``matvec``      reconstruct-then-matmul, the result the GPU matvec is
                  compared with
* ``cpu_path``    the same reconstruct-plus-matmul written with torch CPU ops
                  (what the reference itself would run on host cores); used as
                  the timed CPU baseline only

Each function cites the reference file and lines it follows (paths are inside
the reference project, ``src/mlkit/...``).

Parity pin: the functions here are checked against outputs of the reference
library itself, imported on CPU, on seeded inputs.  Those outputs are stored as
``tests/golden/*.npz`` next to the script that produced them
(``tests/golden/make_golden.py``).

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this package.  The product package (``mlkit_b200``) never does, and it
raises when its CUDA library is missing instead of computing anything on CPU.
"""
