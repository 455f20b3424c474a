"""CPU checkers for the CUDA sampling path (test infrastructure only).

`oracle.port`  — ctypes view of liboracle.so, this repository's C restatement
                 of the reference sampler (oracle/sampler_oracle.c).
`oracle.ref`   — ctypes view of oracle/_ref/libgeist_ref*.so, the reference's own
                 src/engine/sampler.c compiled unmodified (None when not built).

`oracle.ref_drafter` — the reference's own n-gram drafter out of src/engine/session.c
                 (oracle/ref_drafter_harness.c; None when not built).

Only tests/, the smoke check and the bench's CPU legs may import this package;
the product library never does.
"""
from .binding import port, ref, ref_release, ref_drafter, build  # noqa: F401
