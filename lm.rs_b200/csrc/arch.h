// arch.h -- models that come as a folder (config.json + model.safetensors) instead of an LMRS file.  config.json names
// its "architecture"; a registry maps that name to a factory, and the handle behind the C ABI of include/lmrs_b200.h
// drives whatever the factory returns through this interface: the decode step the greedy sampler and the generate loop
// use, and the many-token step that prompts (whole or in portions) go through.  Both run on the model's own KV cache,
// addressed by position like the cache of the LMRS models.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "json.h"

namespace lmrs {

struct StepParams;   // common.cuh: (token, pos, ...) of a decode step in device memory

enum ArchDtype { ARCH_BF16 = 0, ARCH_F32 = 1 };   // bf16 operands with f32 accumulation | everything in true f32

struct ArchOptions {
    int dtype = ARCH_BF16;
    uint32_t max_tokens = 0;   // positions the cache holds (0: the model's default)
    int device = 0;
    int sms = 148;
};

struct ArchInfo {
    std::string architecture;
    uint32_t vocab = 0, width = 0, n_layers = 0, max_tokens = 0;
    uint32_t heads = 0, kv_heads = 0, head_dim = 0, ff = 0;   // of the first layer (informational)
    int dtype = ARCH_BF16;
    float eps = 0.0f;
    int model_type = 3;   // what the handle reports in args.model_type: 3 Genetar, 4 Tudatar, 5 Rupenex, 6 Badepel
};

class ArchModel {
  public:
    virtual ~ArchModel() {}
    ArchInfo info;
    float* d_logits = nullptr;   // [vocab]: logits of the last decode step
    uint64_t launches = 0;       // kernels launched so far
    std::string error;           // message of the last failed call
    // One decode step, enqueued on `st` without synchronising: token and position are read ON THE DEVICE from *d_step
    // (the greedy sampler's kernel advances them between steps); pos_hint is the host's copy of the position.
    virtual int decode_enqueue(cudaStream_t st, const StepParams* d_step, uint32_t pos_hint) = 0;
    // n tokens at positions pos .. pos+n-1 in one pass; logits of the rows listed in `want` (indices into the n tokens,
    // any order) are written to d_out [n_want][vocab] (device).  Enqueued on `st`, not synchronised.
    virtual int forward_tokens(cudaStream_t st, const uint32_t* tokens, size_t n, uint32_t pos, const uint32_t* want,
                               size_t n_want, float* d_out) = 0;
    // test access: the residual stream after every layer of the last forward_tokens call, [n_layers][n][width] (host)
    virtual int read_layer_outputs(cudaStream_t st, float* out, size_t capacity_floats, size_t* n_floats) = 0;
    virtual void set_keep_layer_outputs(bool on) = 0;
    // test access: cached K and V rows [pos0, pos0+n) of a layer, f32 [n][kv_heads * dim] and [n][kv_heads * vdim]
    virtual int read_kv(cudaStream_t st, uint32_t layer, uint32_t pos0, uint32_t n, float* k_out, float* v_out) = 0;
    // measurement aid: device milliseconds per kernel class of the last forward_tokens / decode call when timing is on
    virtual void set_option(const char* name, int value) = 0;
};

typedef ArchModel* (*ArchFactory)(const std::string& dir, const Json& config, const ArchOptions& opt, std::string& err);
void arch_register(const char* architecture, ArchFactory f);
// reads <dir>/config.json and builds the model its "architecture" names; nullptr + err on failure
ArchModel* arch_open(const std::string& dir, const ArchOptions& opt, std::string& err);
bool arch_is_model_dir(const std::string& path);

struct ArchRegistrar {
    ArchRegistrar(const char* architecture, ArchFactory f) { arch_register(architecture, f); }
};

}  // namespace lmrs
