"""B200 (sm_100a) implementation of the int8-quantised linear layer and fp16 decode GEMV of
OpenBMB/cpm_kernels, behind that package's own ``kernels`` / ``torch`` interfaces.

Sub-packages (mirroring the reference's layout for this path):

* ``library``  -- ctypes binding of the C-ABI shim ``libcpmk_b200.so`` (replaces library/cublaslt.py
  and the fatbin loader of kernels/base.py);
* ``device``   -- current-device query and the compute-capability gate;
* ``kernels``  -- ``gemm_*`` / ``gemv_*`` with the reference's signatures: raw device addresses,
  sizes, a ``cudaStream_t``;
* ``torch``    -- ``bmm`` and the ``GEMMInt8`` autograd function;
* ``sharded``  -- column-parallel (N-sharded) linear over ``torch.distributed``.

Importing ``kernels`` or ``torch`` loads the CUDA library and raises if it has not been built
(``python -m cpm_kernels_b200.build``); there is no CPU fallback.
"""
__version__ = "0.1.0"
