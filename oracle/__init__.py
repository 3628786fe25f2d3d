"""CPU oracle for the sparse-convolution hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package may import this folder: only ``tests/``, the
smoke check in ``__graft_entry__`` and the CPU-baseline / reference arms of
``bench.py`` do, and there only as the checker or as the timed CPU baseline.

Contents
--------
``kernel_map.py``   NumPy restatement of the reference's coordinate hashing,
                    kernel-map search/compaction, stride-2 coordinate
                    down-sampling and Morton code (reference: CUDA sources that
                    only run through CuPy on a GPU).
``sparse_conv.py``  torch-CPU restatement of the reference's explicit-GEMM
                    forward, the BatchNorm/ReLU/residual chain and the
                    MinkUNet-34 forward built from them.
``ref_build.py``    recipe that compiles the reference's own self-contained
                    kernel sources (hash table, kernel map, Morton code) as host
                    C++ into ``oracle/_ref/`` through a small shim of CUDA
                    builtins; ``ref_loader.py`` binds them with ctypes and also
                    imports the reference's pure-torch Python functions with the
                    GPU-only dependencies stubbed.

Parity status
-------------
* Kernel map, hash search, Morton code: PINNED — ``kernel_map.py`` is checked
  against the reference's own kernel code compiled for the host
  (``oracle/_ref``) and against golden vectors generated from it
  (``tests/golden``).
* Explicit-GEMM convolution: PINNED — ``sparse_conv.py`` is checked against the
  reference's ``_explicit_gemm_forward_logic`` run on CPU tensors and against
  golden vectors generated from it.
* Dilated windows and custom window centres: PINNED — ``kernel_map_found`` with a
  dilation / centre equals the reference's offset-list kernel
  (``kernel_map_offset_*``) run on its own ``kernel_offsets_from_size`` lists
  (``tests/golden/kmap_extra.npz``).
* Output support of a generative convolution (``expand_coords``): pinned as a SET
  against the reference's expansion loop run with its own hash-search kernel.
* Window reductions (``sparse_conv.window_reduce``): pinned to the reference's
  ``IntSearchResult.to_csr`` + ``row_reduction`` with ``torch.segment_reduce``
  standing in for ``torch_scatter.segment_csr`` (third-party, not installed here).
* Stride-2 output coordinates: pinned as a SET (the reference's row order is
  run-to-run nondeterministic); compared after lexicographic sorting.
* CUTLASS implicit GEMM: third-party arithmetic absent from the reference tree
  (un-vendored submodule, commit not recoverable); its only value-level pin in
  the reference's tests is "close to explicit GEMM", which is the pin used here.
"""
