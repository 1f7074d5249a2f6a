"""Modules under the reference's own module names.  Put this directory on sys.path and the
reference's test and benchmark scripts (`import nvfp4_gemm as G`, `import nvfp4_cuda as C`,
`from nvfp4_train import FP4Linear, mark_step`) run against the B200 kernels unchanged."""
