// Token embedding: ids -> rows of the table, written as the float32 residual stream.
// Reference: bn_model_embed_token bounds-checks the id, zero-fills and logs on a bad
// one, and converts the row to float32 (src/model_embed.c:6-28).
#include "common.cuh"

template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                                    float* __restrict__ out, int width, int vocab, float scale,
                                    int* __restrict__ bad_token) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  int t = blockIdx.x;
  int id = tokens[t];
  float* o = out + (size_t)t * width;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicExch(bad_token, 1);
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = to_f32<T>(row[i]) * scale;
}

// bad_token: one int on the device, set to 1 when an id lies outside [0, vocab).
extern "C" int bn_embed_gather(const void* table, int table_dtype, const int* tokens, float* out,
                               int n_tokens, int width, int vocab, float scale, int* bad_token,
                               cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (width <= 0 || vocab <= 0) return BN_ERR_BAD_ARG;
  int threads = width >= 1024 ? 256 : 128;
  if (table_dtype == BN_F32)
    BN_LAUNCH((embed_gather_kernel<float>), n_tokens, threads, 0, stream, (const float*)table, tokens, out, width, vocab, scale, bad_token);
  else if (table_dtype == BN_BF16)
    BN_LAUNCH((embed_gather_kernel<__nv_bfloat16>), n_tokens, threads, 0, stream, (const __nv_bfloat16*)table, tokens, out, width, vocab, scale, bad_token);
  else
    return BN_ERR_BAD_ARG;
  BN_CHECK_LAUNCH();
  return BN_OK;
}
