"""The kernel modules that the tests need beyond the package's defaults: attention at the tiny
configurations' head sizes and at those of the reference's op tests, and the test build of the tensor-core product.  A build step may compile them ahead of the tests; a test that meets
a module that is not built compiles it itself at first use."""

TEST_MODULES = [
    *[("attention_simt.cu", {"LLB_HEAD_DIM": d}) for d in (4, 8, 10, 16, 20, 24, 32, 48, 80, 160)],
    *[("attention_mma.cu", {"LLB_HEAD_DIM": d}) for d in (16, 32, 48, 80)],
    # keys and values of different widths, and a head size that is no multiple of 4 (test_gpu_vumezen.py)
    *[("attention_simt.cu", {"LLB_HEAD_DIM": k, "LLB_VALUE_DIM": v}) for k, v in ((16, 24), (32, 16), (48, 32))],
    ("attention_simt.cu", {"LLB_HEAD_DIM": 18}), ("attention_simt.cu", {"LLB_HEAD_DIM": 7, "LLB_VALUE_DIM": 5}),
    # latent attention: cache rows (latent + rotated part) whose leading elements are the values (test_gpu_nubedra.py)
    *[("attention_simt.cu", {"LLB_HEAD_DIM": k, "LLB_VALUE_DIM": v}) for k, v in ((40, 24), (48, 40), (28, 18), (28, 20), (9, 7), (272, 264), (32, 24), (56, 40), (14, 10), (8, 6), (600, 560))],
    # attention with a distance penalty, and latent rows without a query latent (test_gpu_zedirax.py)
    *[("attention_simt.cu", {"LLB_HEAD_DIM": k, "LLB_VALUE_DIM": v}) for k, v in ((18, 10), (6, 14), (6, 10), (5, 3), (32, 20), (28, 12), (13, 9), (9, 5), (300, 300))],
    # chunks, two score maps and pooled blocks (test_gpu_zetalorn.py)
    *[("attention_simt.cu", {"LLB_HEAD_DIM": k, "LLB_VALUE_DIM": v}) for k, v in ((24, 8), (10, 6), (16, 8), (12, 20), (16, 32), (32, 64))],
    ("attention_simt.cu", {"LLB_HEAD_DIM": 12}),
    # the build in which a bounded wait can be made to run out (test_gpu_kernels.py)
    ("gemm_tc.cu", {"LLB_WAIT_LIMIT": 4096, "LLB_TEST_STALL": 1}),
]
