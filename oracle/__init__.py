"""CPU oracle for the DCNv4 / FlashDeformAttn operator path.

TEST INFRASTRUCTURE ONLY: the checker the CUDA kernels are compared against.
Only the test suite, the smoke check and the benchmark's CPU-baseline leg may
import this package; the product package never does.

* `oracle.cref`      -- ctypes front end of the plain-C restatement (`dcn_oracle.c`),
                        fp32 coordinates / fp64 accumulation, also emits the integer
                        corner indices every sampling point selects.
* `oracle.torch_core`-- an independent grid_sample-based PyTorch formulation of the
                        same four ops (forward; backward through autograd).  It is
                        the second opinion that pins the C restatement and the CPU
                        implementation timed as the CPU baseline.
* `oracle.inputs`    -- seeded synthetic inputs with the benchmark configurations' shapes
                        and value distributions.
"""
