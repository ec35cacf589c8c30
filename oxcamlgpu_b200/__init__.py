"""oxcamlgpu_b200 -- B200-native dense GEMM path of the OxCaml GPU compiler.

The product is ``liboxgpu_b200.so`` (CUDA kernels for sm_100a behind a C ABI,
``include/oxgpu_b200.h``).  This package is the thin host side above it:

* ``catalog``  -- mirror of the reference's ``Gemm_catalog`` (test/gemm_catalog.ml)
* ``gemm``     -- launcher mirroring test/hardware/run_gemm_h100.cu and
                  bench/bench.py (tensor maps, catalog entry points, buffers)
* ``sharded``  -- column-sharded multi-GPU driver (one process per GPU)
* ``synth``    -- seeded synthetic operands
* ``build``    -- the nvcc recipe

Nothing here computes a GEMM on the CPU; without the CUDA library every
compute call raises.  Submodules are imported on demand.
"""
