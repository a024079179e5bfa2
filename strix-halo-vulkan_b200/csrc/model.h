// The checkpoint on the device: tensors by name plus the per-layer view the graph walks.
#pragma once
#include <map>
#include <string>
#include <vector>

#include "../../include/b200_llm.h"
#include "common.cuh"

namespace b200 {

struct LayerW {
  bool is_attn = false;
  DTensor attn_norm, ffn_norm;
  DTensor qkv, z, alpha, beta, conv1d, ssm_a, dt_bias, ssm_norm, ssm_out;   // gated DeltaNet
  DTensor q, k, v, o, q_norm, k_norm;                                       // gated GQA attention
  DTensor router, sh_gate_inp, gate_exps, up_exps, down_exps, gate_sh, up_sh, down_sh;
  DTensor enorm, hnorm, eh_proj, head_norm;                                 // draft layer only
};

struct Model {
  b200_config c{};
  int device = 0;
  bool finalized = false;
  std::map<std::string, DTensor> tensors;
  std::map<std::string, std::vector<int64_t>> dims;
  std::vector<void*> allocs;
  std::vector<LayerW> layers;  // n_layer (+1 draft)
  DTensor token_embd, output, output_norm;
  int64_t weight_bytes = 0;

  ~Model();
  int alloc_tensor(const std::string& name, uint32_t type, uint32_t n_dims, const int64_t* d, DTensor* out);
  int add_host(const std::string& name, uint32_t type, uint32_t n_dims, const int64_t* d, const void* host);
  int add_synthetic(const std::string& name, uint32_t type, uint32_t n_dims, const int64_t* d, uint64_t seed, int rule, float p0, float p1);
  int finalize();
  int read_tensor(const std::string& name, void* dst, int64_t nbytes) const;
};

int load_gguf_into(const char* path, int device, Model* m);

// device-side synthetic values + quantiser (synth.cu)
int synth_fill(float* dst, int64_t n, uint64_t seed, int rule, float p0, float p1, cudaStream_t st);
int quantize_rows_device(uint32_t type, const float* src, int64_t rows, int64_t k, uint8_t* gguf_dst, cudaStream_t st);

// projection through a file-scope device staging array (static_scratch.cu)
int qgemv_static(uint32_t type, const void* dev_w, int64_t rows, int64_t k, const float* dev_x, int32_t m, float* dev_y);

}  // namespace b200
