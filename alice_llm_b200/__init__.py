"""B200 (sm_100a) quantized-matvec decode path for ALICE-LLM: hand-written CUDA kernels behind
a C ABI (include/alice_cuda.h), with a host-side mirror of the reference's entry points.

  alice_llm_b200.gguf   signatures of src/gguf.rs (quantized_matvec, quantize_row_q8_k, ...)
  alice_llm_b200.gpu    GpuEngine / GpuPass / GpuWeightBuffer of src/gpu.rs
  alice_llm_b200.synth  seeded synthetic weights in the GGUF block formats

There is no CPU fallback: importing works anywhere, computing needs a CUDA device.
"""
__version__ = "0.1.0"
