// Library-wide state: launch counter, device status word, tensor-map encoder.
#include "common.cuh"

#include <stdio.h>
#include <string.h>
#include <stdlib.h>

#include <mutex>
#include <unordered_map>

namespace tlm {

unsigned long long g_launches = 0;
int g_deterministic = 0;

static unsigned int* g_status_host = nullptr;
static unsigned int* g_status_dev = nullptr;

unsigned int* status_word() {
  if (g_status_dev == nullptr) {
    if (cudaHostAlloc((void**)&g_status_host, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) return nullptr;
    *g_status_host = 0;
    if (cudaHostGetDevicePointer((void**)&g_status_dev, g_status_host, 0) != cudaSuccess) return nullptr;
  }
  return g_status_dev;
}

unsigned int read_status(bool clear) {
  if (g_status_host == nullptr) return 0;
  unsigned int v = *(volatile unsigned int*)g_status_host;
  if (clear && v != 0) *(volatile unsigned int*)g_status_host = 0;
  return v;
}

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) return nullptr;
    fn = (EncodeTiledFn)p;
  }
  return fn;
}

// Encoded maps are pure functions of (base, dims, strides, box); training re-launches the same
// few hundred operand shapes on the same addresses every step, so they are memoised.
struct TmapKey {
  uint64_t v[16];
  bool operator==(const TmapKey& o) const { return memcmp(v, o.v, sizeof(v)) == 0; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (int i = 0; i < 16; ++i) { h ^= k.v[i]; h *= 1099511628211ull; }
    return (size_t)h;
  }
};
static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmap_cache;
static std::mutex g_tmap_mutex;

static int make_tmap(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box);

int make_tmap_bf16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                   const uint32_t* box) {
  return make_tmap(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, rank, dims, strides_bytes, box);
}

int make_tmap_f32(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                  const uint32_t* box) {
  return make_tmap(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, rank, dims, strides_bytes, box);
}

static int make_tmap(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return -1;
  TmapKey key{};
  key.v[0] = (uint64_t)(uintptr_t)base;
  key.v[1] = (uint64_t)rank | ((uint64_t)dtype << 8);
  for (int i = 0; i < rank; ++i) {
    key.v[2 + i] = dims[i];
    key.v[7 + i] = (uint64_t)box[i];
    if (i + 1 < rank) key.v[12 + i] = strides_bytes[i];
  }
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    auto it = g_tmap_cache.find(key);
    if (it != g_tmap_cache.end()) { *map = it->second; return 0; }
  }
  cuuint64_t gdim[5], gstr[4];
  cuuint32_t bdim[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
    if (i + 1 < rank) gstr[i] = strides_bytes[i];
  }
  CUresult r = enc(map, dtype, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bdim,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "tlm: cuTensorMapEncodeTiled failed (%d): rank %d base %p dims", (int)r, rank, base);
    for (int i = 0; i < rank; ++i) fprintf(stderr, " %llu", (unsigned long long)dims[i]);
    fprintf(stderr, " box");
    for (int i = 0; i < rank; ++i) fprintf(stderr, " %u", box[i]);
    fprintf(stderr, "\n");
    return (int)r;
  }
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    if (g_tmap_cache.size() > 65536) g_tmap_cache.clear();
    g_tmap_cache.emplace(key, *map);
  }
  return 0;
}

int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

int attn_head_group(const char* env, long long bytes_per_head, long long budget_bytes, int n_heads) {
  long long g = bytes_per_head > 0 ? budget_bytes / bytes_per_head : 1;
  const char* v = getenv(env);
  if (v != nullptr && atoi(v) > 0) g = atoi(v);
  if (g > n_heads) g = n_heads;
  return g < 1 ? 1 : (int)g;
}

}  // namespace tlm

TLM_API unsigned long long tlm_launch_count() { return tlm::g_launches; }
TLM_API void tlm_reset_launch_count() { tlm::g_launches = 0; }
// Launches that the launchers did not see: a recorded step replayed as a CUDA graph runs the same kernels again.
TLM_API void tlm_add_launch_count(unsigned long long n) { tlm::g_launches += n; }

// Reads (and clears) the status word; 0 = no kernel gave up on a wait. Does not
// synchronise: call after the work of interest has completed.
TLM_API unsigned int tlm_take_device_status() { return tlm::read_status(true); }

TLM_API int tlm_num_sms() { return tlm::num_sms(); }

// Deterministic mode: kernels avoid floating-point atomics whose order depends on scheduling (the split-K
// weight-gradient epilogue). Slower on small outputs; bit-reproducible runs on the same hardware.
TLM_API void tlm_set_deterministic(int on) { tlm::g_deterministic = on; }
TLM_API int tlm_get_deterministic() { return tlm::g_deterministic; }
