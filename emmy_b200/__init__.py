"""B200 (sm_100a) kernels for the quantized-linear operator, behind a C ABI.

`emmy_b200.lib` loads libemmyq.so (built in-tree by `python -m emmy_b200.build`),
`emmy_b200.ops` wraps its entry points for torch tensors, `emmy_b200.linear`
holds the modules that take a checkpoint's tensors under their own names.
There is no CPU path: without the built library, or without a CUDA device,
the operators raise.
"""

__version__ = "0.1.0"
