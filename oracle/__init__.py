"""CPU oracle for the burn-mamba SSM hot path.

TEST INFRASTRUCTURE ONLY.  Nothing under ``oracle/`` is part of the shipped
library: only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` may import or execute it, and there
only as the checker (or as the timed CPU comparison), never as the thing that
is measured as the product.

PARITY UNPINNED.  The reference (swfsql/burn-mamba) is pure Rust over the
un-vendored git dependency ``burn 0.22.0-pre.2`` (rev 1893b608d1c7…); no Rust
toolchain exists where this was written, so the reference cannot be executed,
and the reference's own tests hold no golden vectors, fixtures or seeded known
answers (all of them are unseeded self-consistency properties).  The oracle is
therefore a restatement of the reference's *formulas*, each function citing the
reference file:line it follows, and it is anchored only by the invariants the
reference's tests assert:

* Minimal == Serial SSD variants                  (src/mamba2/ssd/ssd_path/tests.rs:184-336)
* forward == unrolled step                         (src/mamba2/mamba2/tests.rs:202-252,
                                                    src/mamba1/mamba1/tests.rs:216-265,
                                                    src/mamba3/double_ssd/double_ssd/tests.rs:259-307)
* split prefill == full prefill                    (src/mamba2/mamba2/tests.rs:343-392)
* single-SSD == double-SSD                         (src/mamba3/single_ssd/single_ssd/tests.rs:374-428)
* mimo_outer_sum == hand-written loops             (src/mamba3/helpers/tests.rs:13-72)
* angle increment == dt * pi * tanh(rot) at range 1 (src/mamba3/rotation/tests.rs:1238-1248)

plus an independent float64 sequential recurrence (the ``step()`` math unrolled)
used as ground truth for the chunked forms.

Modules:
    numerics  softplus / SiLU / RMSNorm / gated RMSNorm / div_eps / bf16 rounding
    mamba2    chunked SSD (serial + minimal + recurrence), block forward, step
    mamba1    sequential selective scan, block forward, step
    mamba3    trapezoid coefficients, QK-norm, rotation, single/double SSD, step
    backward  analytic Mamba-2 / Mamba-3 SSD gradients + finite differences
    inputs    seeded generators for the benchmark configurations
"""
