"""CPU oracle for the quantized-linear path.

TEST INFRASTRUCTURE ONLY.  This package restates, in numpy and CPU torch, the
arithmetic of the reference's eager "dequantize then matmul" path
(emmy/compiler/loader/quant.py, emmy/compiler/dtype.py, the MoE glue in
emmy/serving/gen_runner.py and emmy/compiler/trace/huggingface.py).  It exists
so that the CUDA kernels can be checked, and so that the reference's CPU path
can be timed next to them.  Nothing in the shipped package imports it: only
the test-suite, the smoke check and the benchmark's CPU-baseline leg do.

Pinning.  The codecs, int4 unpack/dequant, NVFP4 quantize/dequantize, the
static NVFP4 activation round trip and the dynamic FP8 activation rule are
pinned against (a) the known-answer vectors of the reference's own tests and
(b) outputs of the reference's numpy functions themselves, captured into
tests/golden/quant_golden.npz by tests/golden/make_golden.py.

Parity unpinned (the reference has nothing to pin them against):
  * GPTQ act-order (a non-identity g_idx): the reference rejects desc_act
    checkpoints, so `dequant_w4(..., g_idx=...)` follows the published GPTQ
    rule group(k) = g_idx[k] only.
  * expert-parallel all-to-all MoE: the reference shards experts along the
    intermediate axis and all-reduces instead.
"""
