// Handle types and error helpers shared by the translation units that implement the C ABI.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/alice_cuda.h"
#include "gemv_launch.cuh"
#include "q8k.cuh"

struct alice_engine {
    int device = 0;
    int num_sms = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    bool pdl = true;
    int force_rps = 0, force_stages = 0;
    int* status = nullptr;        // device status word
    int* status_host = nullptr;   // pinned host word alice_sync copies it into
    void* scratch = nullptr;      // engine-owned scratch: Q8_K of the current input, or its f32 form
    size_t scratch_bytes = 0;
    void* prep = nullptr;         // engine-owned scratch of the bit-plane kernels: the activation digit table of the current input
    size_t prep_bytes = 0;
    long long wait_limit = 0;          // SM cycles a kernel wait may take (0 = about one second)
    // handles created on the engine keep the struct alive after alice_engine_destroy (which releases everything else)
    int refs = 1;
    bool dead = false;
    // tensor-parallel group (csrc/tp.cu): this engine is rank tp_rank of tp_world, one engine per GPU
    uint32_t tp_rank = 0, tp_world = 1;
    void* tp_comm = nullptr;      // ncclComm_t
};

struct alice_weights {
    alice_engine* e;
    alice::WeightDesc d;
    void* owned_data = nullptr;
    void* owned_scales = nullptr;
};

struct alice_buf {
    alice_engine* e;
    float* p;
    size_t len;
    bool owned;
};

struct alice_q8k {
    alice_engine* e;
    void* base;
    uint32_t cols, batch, nb;
    alice::Q8KLayout lay;
};

// Records the message returned by alice_last_error() for the calling thread; returns `code`.
int alice_fail(int code, const char* fmt, ...);
int alice_cuda_fail(cudaError_t err, const char* what);
alice::LaunchCfg alice_cfg_of(const alice_engine* e);
void alice_engine_retain(alice_engine* e);
void alice_engine_release(alice_engine* e);
