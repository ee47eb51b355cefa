"""Python-side plumbing of the B200 MoE forward path: the ctypes binding of the C ABI, seeded synthetic
inputs, and the expert-parallel driver over torch.distributed.  The compute lives in libxs_moe.so."""
