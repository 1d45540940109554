// Tensor-parallel exchange steps of the decoder.  The reference has no multi-device
// code; this follows the Megatron layout: after each row-parallel projection (o_proj,
// down) the ranks' partial sums [batch, hidden] are added up and added to the residual
// stream, and the vocabulary-sharded logits are gathered.
//
// Two implementations of the sum:
//  * ncclAllReduce (the baseline; NCCL is loaded at run time with dlopen so that a process
//    that already carries an NCCL - e.g. through torch - shares it), followed by the
//    residual add;
//  * a one-shot kernel over peer memory: the projection writes its partial straight into a
//    buffer that every rank has mapped (cudaIpc), a flag per rank announces it, and each
//    rank reads all partials over NVLink with plain loads, adds them in rank order (so every
//    rank holds bit-identical sums) and applies the residual - one launch, no extra
//    pass over the data.  Every wait on a peer's flag is bounded; when it runs out the
//    kernel raises an error word and returns.
#include <dlfcn.h>

#include <cstring>
#include <vector>

#include "tp.cuh"

namespace tb {

namespace {

struct NcclId { char internal[128]; };
typedef void* nccl_comm_t;
typedef int (*fn_get_unique_id)(NcclId*);
typedef int (*fn_comm_init_rank)(nccl_comm_t*, int, NcclId, int);
typedef int (*fn_comm_destroy)(nccl_comm_t);
typedef int (*fn_all_reduce)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t);
typedef int (*fn_all_gather)(const void*, void*, size_t, int, nccl_comm_t, cudaStream_t);
typedef int (*fn_group)(void);
typedef const char* (*fn_err_string)(int);

struct NcclApi {
  void* lib = nullptr;
  fn_get_unique_id get_unique_id = nullptr;
  fn_comm_init_rank comm_init_rank = nullptr;
  fn_comm_destroy comm_destroy = nullptr;
  fn_all_reduce all_reduce = nullptr;
  fn_all_gather all_gather = nullptr;
  fn_group group_start = nullptr, group_end = nullptr;
  fn_err_string err_string = nullptr;
};

constexpr int kNcclFloat32 = 7, kNcclSum = 0;

NcclApi* nccl() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return api.lib ? &api : nullptr;
  tried = true;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    api.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (api.lib) break;
  }
  if (!api.lib) return nullptr;
  api.get_unique_id = (fn_get_unique_id)dlsym(api.lib, "ncclGetUniqueId");
  api.comm_init_rank = (fn_comm_init_rank)dlsym(api.lib, "ncclCommInitRank");
  api.comm_destroy = (fn_comm_destroy)dlsym(api.lib, "ncclCommDestroy");
  api.all_reduce = (fn_all_reduce)dlsym(api.lib, "ncclAllReduce");
  api.all_gather = (fn_all_gather)dlsym(api.lib, "ncclAllGather");
  api.group_start = (fn_group)dlsym(api.lib, "ncclGroupStart");
  api.group_end = (fn_group)dlsym(api.lib, "ncclGroupEnd");
  api.err_string = (fn_err_string)dlsym(api.lib, "ncclGetErrorString");
  if (!api.get_unique_id || !api.comm_init_rank || !api.comm_destroy || !api.all_reduce || !api.all_gather ||
      !api.group_start || !api.group_end) {
    dlclose(api.lib);
    api.lib = nullptr;
    return nullptr;
  }
  return &api;
}

#define TB_NCCL_TRY(api, expr)                                                          \
  do {                                                                                  \
    int _r = (expr);                                                                    \
    if (_r != 0)                                                                        \
      return fail(TB_ERR_NCCL, "%s failed: %s", #expr,                                  \
                  (api)->err_string ? (api)->err_string(_r) : "nccl error");            \
  } while (0)

constexpr int kMaxRanks = 8;
constexpr int kLLLines = 8192;     // float2 lines per rank in the low-latency receive area (16384 floats)
constexpr long long kPeerWaitCycles = 20000000000ll;  // ~10 s: ranks may be apart by a graph instantiation
long long g_peer_wait_cycles = 0;   // test hook: a shorter limit (0 = the default above)

struct PeerArgs {
  const float* bufs[kMaxRanks];  // every rank's partial for this call, [count] floats
  uint32_t* my_flags;            // flags[src]: written by rank src (over NVLink)
  uint32_t* peer_flags[kMaxRanks];
  uint32_t* epoch;               // device word: number of completed exchanges
  int* done_ctas;                // ticket for the epoch increment
  int* err;
  int* host_fault;               // optional host-mapped word: set with err, read by the host without a copy
  long long wait_cycles;         // limit of the wait for the peers
  float* x;                      // residual stream, updated in place
  int rank, size;
  int count4;                    // float4 elements
};

__device__ __forceinline__ float4 ld_volatile_f4(const float4* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// x += sum over ranks of partial_r, partial_r read from rank r's memory.
__global__ void __launch_bounds__(1024) peer_allreduce_residual_kernel(const PeerArgs a) {
  __shared__ int s_ok;
  const uint32_t want = *a.epoch + 1;
  if (threadIdx.x == 0) {
    s_ok = 1;
    if (blockIdx.x == 0) {
      // My partial was written by the previous kernel on this stream: publish it.
      __threadfence_system();
      for (int r = 0; r < a.size; ++r) st_release_sys(a.peer_flags[r] + a.rank, want);
    }
  }
  __syncthreads();
  if (threadIdx.x < a.size) {
    const long long t0 = clock64();
    while (ld_acquire_sys(a.my_flags + threadIdx.x) < want) {
      if (clock64() - t0 > a.wait_cycles) {  // a peer never arrived: give up, flag the error
        s_ok = 0;
        atomicExch(a.err, 1);
        if (a.host_fault) *reinterpret_cast<volatile int*>(a.host_fault) = 1;
        break;
      }
    }
  }
  __syncthreads();
  if (s_ok) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < a.count4; i += gridDim.x * blockDim.x) {
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < a.size; ++r) {
        const float4 v = ld_volatile_f4(reinterpret_cast<const float4*>(a.bufs[r]) + i);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
      float4 xv = reinterpret_cast<float4*>(a.x)[i];
      xv.x += s.x; xv.y += s.y; xv.z += s.z; xv.w += s.w;
      reinterpret_cast<float4*>(a.x)[i] = xv;
    }
  }
  // the last CTA closes the exchange
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(a.done_ctas, 1) == (int)gridDim.x - 1) {
      *a.done_ctas = 0;
      *a.epoch = want;
    }
  }
}

// ------------------------------------------------------------------------------------------
// Low-latency form for small exchanges (one decode step of a few sequences): every 16-byte line
// that crosses NVLink carries two floats and, twice, the number of the exchange.  A rank pushes
// its partial into a receive area in every peer's memory (posted stores, one way) and then polls
// its own receive area line by line until both copies of the number have arrived - no fence, no
// separate flag, no read across the link.  A line is written with one 16-byte store; should the
// two halves become visible apart, the second copy of the number is still missing and the poll
// goes on.  Sums are taken in rank order on every rank (bit-identical x everywhere).  Optionally
// also writes x times the next norm's weights and the sums of squares of x per 8 elements (the
// split RMSNorm of the decoder).  One CTA; the exchange number lives in device memory so that
// the launch can be replayed from a CUDA graph.
// ------------------------------------------------------------------------------------------
struct LLArgs {
  const float* partial;             // this rank's partial, [count] floats (local)
  uint4* my_recv;                   // [size][lines_cap] lines written by the peers
  uint4* peer_recv[kMaxRanks];      // the same area in every peer's memory
  uint32_t* epoch;
  int* err;
  int* host_fault;
  long long wait_cycles;
  float* x;
  const float* scale_w;             // optional: next norm's weights [count]
  float* out_scaled;                // optional: x * scale_w
  float* out_ss8;                   // optional: sums of x^2 over 8 consecutive elements
  int rank, size;
  int lines, lines_cap;             // float2 lines in use / per rank in the receive area
};

__global__ void __launch_bounds__(1024) ll_allreduce_residual_kernel(const LLArgs a) {
  const uint32_t want = *a.epoch + 1;
  const float2* mine = reinterpret_cast<const float2*>(a.partial);
  for (int i = threadIdx.x; i < a.lines; i += blockDim.x) {
    const float2 v = mine[i];
    const uint4 line = make_uint4(__float_as_uint(v.x), want, __float_as_uint(v.y), want);
    for (int r = 0; r < a.size; ++r) {
      if (r == a.rank) continue;
      uint4* dst = a.peer_recv[r] + (size_t)a.rank * a.lines_cap + i;
      asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(line.x), "r"(line.y), "r"(line.z), "r"(line.w) : "memory");
    }
  }
  bool ok = true;
  const long long t0 = clock64();
  const int rounds = (a.lines + (int)blockDim.x - 1) / (int)blockDim.x;
  for (int k = 0; k < rounds; ++k) {
    const int i = k * blockDim.x + threadIdx.x;
    const bool live = i < a.lines;
    float2 s = make_float2(0.f, 0.f);
    if (live) {
      for (int r = 0; r < a.size; ++r) {
        float2 v;
        if (r == a.rank) {
          v = mine[i];
        } else {
          const uint4* src = a.my_recv + (size_t)r * a.lines_cap + i;
          uint4 line;
          for (uint32_t spin = 0;; ++spin) {
            asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(line.x), "=r"(line.y), "=r"(line.z), "=r"(line.w) : "l"(src) : "memory");
            if (line.y == want && line.w == want) break;
            if (!ok || ((spin & 1023) == 1023 && clock64() - t0 > a.wait_cycles)) {  // the peer never arrived
              if (ok) {
                atomicExch(a.err, 1);
                if (a.host_fault) *reinterpret_cast<volatile int*>(a.host_fault) = 1;
              }
              ok = false;
              break;
            }
          }
          v = make_float2(__uint_as_float(line.x), __uint_as_float(line.z));
        }
        s.x += v.x;
        s.y += v.y;
      }
    }
    float2 xv = make_float2(0.f, 0.f);
    if (live) {
      xv = reinterpret_cast<float2*>(a.x)[i];
      xv.x += s.x;
      xv.y += s.y;
      reinterpret_cast<float2*>(a.x)[i] = xv;
      if (a.out_scaled != nullptr) {
        const float2 w = reinterpret_cast<const float2*>(a.scale_w)[i];
        reinterpret_cast<float2*>(a.out_scaled)[i] = make_float2(xv.x * w.x, xv.y * w.y);
      }
    }
    if (a.out_ss8 != nullptr) {  // 8 consecutive elements = 4 consecutive lanes
      float sq = xv.x * xv.x + xv.y * xv.y;
      sq += __shfl_xor_sync(0xffffffffu, sq, 1);
      sq += __shfl_xor_sync(0xffffffffu, sq, 2);
      if (live && (threadIdx.x & 3) == 0) a.out_ss8[i >> 2] = sq;
    }
  }
  __syncthreads();  // every thread has read the exchange number
  if (threadIdx.x == 0) *a.epoch = want;
}

__global__ void add_inplace_kernel(float* __restrict__ x, const float* __restrict__ y, int n4) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n4) {
    float4 a = reinterpret_cast<float4*>(x)[i];
    const float4 b = reinterpret_cast<const float4*>(y)[i];
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    reinterpret_cast<float4*>(x)[i] = a;
  }
}

}  // namespace

struct TpState {
  int rank = 0, size = 1;
  nccl_comm_t comm = nullptr;
  bool fused = false;
  size_t max_count = 0;       // floats per partial
  // fused path
  int* host_fault = nullptr;  // host-mapped word the exchange kernels raise when a bounded wait runs out
  char* block = nullptr;      // my shared block: [2][max_count] floats | flags | epoch | ticket | err
  char* peer_block[kMaxRanks] = {};
  size_t flags_off = 0;
  int calls = 0;              // host-side call parity selects the buffer a projection writes to
  size_t ll_off = 0;          // low-latency receive area: [2][size][kLLLines] lines of 16 bytes
  int ll_calls = 0;
  // areas of the persistent step kernel (one launch per token, exchanges inside the kernel)
  size_t step_recv_off = 0;   // [2][size][hidden] entries of 8 bytes {partial, exchange number}
  size_t step_logits_off = 0; // [logit_floats] floats: every rank stores its slice into every peer's copy
  size_t hidden = 0, logit_floats = 0;
  float* reduced = nullptr;   // NCCL path: the summed partial
};

float* tp_partial_buffer(TpState* st, float* fallback) {
  if (!st || !st->fused) return fallback;
  return reinterpret_cast<float*>(st->block) + (size_t)(st->calls & 1) * st->max_count;
}

bool tp_low_latency(const TpState* st, int batch, int64_t hidden) {
  const size_t count = (size_t)batch * hidden;
  return st && st->fused && (count & 7) == 0 && count / 2 <= (size_t)kLLLines;
}

tb_status tp_allreduce_residual(TpState* st, const float* partial, float* x, int batch, int64_t hidden,
                                cudaStream_t stream, int* launches, const float* scale_w, float* out_scaled,
                                float* out_ss8) {
  if (!st || !st->comm) return fail(TB_ERR_NCCL, "tensor-parallel decoder used before tb_decoder_tp_init");
  const size_t count = (size_t)batch * hidden;
  if (count > st->max_count || (count & 3)) return fail(TB_ERR_SHAPE, "tp all-reduce: %zu elements", count);
  if ((out_scaled || out_ss8) && !tp_low_latency(st, batch, hidden))
    return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: the split RMSNorm outputs need the low-latency exchange");
  if (tp_low_latency(st, batch, hidden)) {
    if (partial != reinterpret_cast<const float*>(st->block) + (size_t)(st->calls & 1) * st->max_count)
      return fail(TB_ERR_ARG, "tp all-reduce: the partial must be written to tp_partial_buffer()");
    st->calls++;
    const int slot = st->ll_calls & 1;
    st->ll_calls++;
    LLArgs a;
    a.partial = partial;
    const size_t slot_lines = (size_t)slot * st->size * kLLLines;
    for (int r = 0; r < st->size; ++r)
      a.peer_recv[r] = reinterpret_cast<uint4*>(st->peer_block[r] + st->ll_off) + slot_lines;
    a.my_recv = reinterpret_cast<uint4*>(st->block + st->ll_off) + slot_lines;
    uint32_t* words = reinterpret_cast<uint32_t*>(st->block + st->flags_off);
    a.epoch = words + 20;
    a.err = reinterpret_cast<int*>(words + 18);
    a.host_fault = st->host_fault;
    a.wait_cycles = g_peer_wait_cycles > 0 ? g_peer_wait_cycles : kPeerWaitCycles;
    a.x = x;
    a.scale_w = scale_w; a.out_scaled = out_scaled; a.out_ss8 = out_ss8;
    a.rank = st->rank; a.size = st->size;
    a.lines = (int)(count / 2); a.lines_cap = kLLLines;
    ll_allreduce_residual_kernel<<<1, 1024, 0, stream>>>(a);
    TB_CUDA_TRY(cudaGetLastError());
    if (launches) ++*launches;
    return TB_OK;
  }
  if (st->fused) {
    const int slot = st->calls & 1;
    st->calls++;
    PeerArgs a;
    for (int r = 0; r < st->size; ++r) {
      a.bufs[r] = reinterpret_cast<const float*>(st->peer_block[r]) + (size_t)slot * st->max_count;
      a.peer_flags[r] = reinterpret_cast<uint32_t*>(st->peer_block[r] + st->flags_off);
    }
    if (partial != a.bufs[st->rank]) return fail(TB_ERR_ARG, "tp all-reduce: the partial must be written to tp_partial_buffer()");
    uint32_t* words = reinterpret_cast<uint32_t*>(st->block + st->flags_off);
    a.my_flags = words;
    a.epoch = words + 16;
    a.done_ctas = reinterpret_cast<int*>(words + 17);
    a.err = reinterpret_cast<int*>(words + 18);
    a.host_fault = st->host_fault;
    a.wait_cycles = g_peer_wait_cycles > 0 ? g_peer_wait_cycles : kPeerWaitCycles;
    a.x = x;
    a.rank = st->rank; a.size = st->size;
    a.count4 = (int)(count / 4);
    int grid = (a.count4 + 1023) / 1024;
    if (grid > 16) grid = 16;
    peer_allreduce_residual_kernel<<<grid, 1024, 0, stream>>>(a);
    TB_CUDA_TRY(cudaGetLastError());
    if (launches) ++*launches;
    return TB_OK;
  }
  NcclApi* api = nccl();
  TB_NCCL_TRY(api, api->all_reduce(partial, st->reduced, count, kNcclFloat32, kNcclSum, st->comm, stream));
  const int n4 = (int)(count / 4);
  add_inplace_kernel<<<(n4 + 255) / 256, 256, 0, stream>>>(x, st->reduced, n4);
  TB_CUDA_TRY(cudaGetLastError());
  if (launches) *launches += 2;
  return TB_OK;
}

tb_status tp_allgather_logits(TpState* st, const float* logits_l, float* logits, int batch,
                              int64_t v_local, cudaStream_t stream, int* launches) {
  if (!st || !st->comm) return fail(TB_ERR_NCCL, "tensor-parallel decoder used before tb_decoder_tp_init");
  NcclApi* api = nccl();
  const int64_t v = v_local * st->size;
  if (batch > 1) TB_NCCL_TRY(api, api->group_start());
  for (int b = 0; b < batch; ++b)
    TB_NCCL_TRY(api, api->all_gather(logits_l + (size_t)b * v_local, logits + (size_t)b * v, (size_t)v_local,
                                     kNcclFloat32, st->comm, stream));
  if (batch > 1) TB_NCCL_TRY(api, api->group_end());
  if (launches) ++*launches;
  return TB_OK;
}

// Peer-visible areas of the persistent step kernel: for every rank the receive area of the
// in-kernel exchanges, the gathered logits and the word where peers announce their logit slices;
// this rank's exchange counter and error word.
bool tp_step_areas(TpState* st, StepTp* t) {
  if (!st || !st->fused || st->hidden == 0) return false;
  t->rank = st->rank; t->size = st->size; t->hidden = (int)st->hidden;
  for (int r = 0; r < st->size; ++r) {
    t->recv[r] = reinterpret_cast<uint2*>(st->peer_block[r] + st->step_recv_off);
    t->logits[r] = reinterpret_cast<float*>(st->peer_block[r] + st->step_logits_off);
    t->flags[r] = reinterpret_cast<uint32_t*>(st->peer_block[r] + st->flags_off) + 32;   // words 32..39: one per source rank
  }
  uint32_t* words = reinterpret_cast<uint32_t*>(st->block + st->flags_off);
  t->epoch = words + 24;
  t->err = reinterpret_cast<int*>(words + 18);
  return true;
}
float* tp_step_logits(TpState* st) {
  return st && st->fused && st->logit_floats ? reinterpret_cast<float*>(st->block + st->step_logits_off) : nullptr;
}

void tp_set_wait_limit(long long cycles) { g_peer_wait_cycles = cycles; }

void tp_set_host_fault(TpState* st, int* device_pointer_of_mapped_word) {
  if (st) st->host_fault = device_pointer_of_mapped_word;
}

int tp_error_flag(TpState* st) {
  if (!st || !st->fused) return 0;
  int v = 0;
  if (cudaMemcpy(&v, st->block + st->flags_off + 18 * sizeof(uint32_t), sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return v;
}

void tp_destroy(TpState* st) {
  if (!st) return;
  for (int r = 0; r < st->size; ++r)
    if (r != st->rank && st->peer_block[r]) cudaIpcCloseMemHandle(st->peer_block[r]);
  cudaFree(st->block);
  cudaFree(st->reduced);
  if (st->comm) {
    NcclApi* api = nccl();
    if (api) api->comm_destroy(st->comm);
  }
  delete st;
}

tb_status tp_create(TpState** out, int rank, int size, const uint8_t id[128], size_t max_count,
                    tb_allgather_fn allgather, void* user, bool nccl_only, size_t hidden, size_t logit_floats) {
  *out = nullptr;
  if (size < 2 || size > kMaxRanks || rank < 0 || rank >= size) return fail(TB_ERR_ARG, "tensor parallel size %d / rank %d (supported: 2..%d ranks)", size, rank, kMaxRanks);
  NcclApi* api = nccl();
  if (!api) return fail(TB_ERR_NCCL, "libnccl.so.2 could not be loaded: %s", dlerror());
  TpState* st = new TpState();
  st->rank = rank; st->size = size; st->max_count = (max_count + 3) & ~(size_t)3;
  NcclId nid;
  memcpy(nid.internal, id, 128);
  int r = api->comm_init_rank(&st->comm, size, nid, rank);
  if (r != 0) {
    delete st;
    return fail(TB_ERR_NCCL, "ncclCommInitRank failed: %s", api->err_string ? api->err_string(r) : "?");
  }
  auto bail = [&](tb_status s) { tp_destroy(st); return s; };
  cudaError_t e = cudaMalloc(&st->reduced, st->max_count * sizeof(float));
  if (e != cudaSuccess) return bail(fail(TB_ERR_OOM, "tp: %s", cudaGetErrorString(e)));
  if (allgather && !nccl_only) {
    st->flags_off = 2 * st->max_count * sizeof(float);
    st->ll_off = st->flags_off + 256;
    st->hidden = hidden; st->logit_floats = logit_floats;
    st->step_recv_off = st->ll_off + (size_t)2 * size * kLLLines * sizeof(uint4);
    st->step_logits_off = st->step_recv_off + (((size_t)2 * size * hidden * 8 + 255) & ~(size_t)255);
    const size_t bytes = st->step_logits_off + ((logit_floats * sizeof(float) + 255) & ~(size_t)255);
    e = cudaMalloc(&st->block, bytes);
    if (e != cudaSuccess) return bail(fail(TB_ERR_OOM, "tp: %s", cudaGetErrorString(e)));
    cudaMemset(st->block, 0, bytes);
    cudaDeviceSynchronize();
    cudaIpcMemHandle_t mine;
    e = cudaIpcGetMemHandle(&mine, st->block);
    if (e != cudaSuccess) return bail(fail(TB_ERR_CUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e)));
    std::vector<cudaIpcMemHandle_t> all(size);
    if (allgather(user, &mine, all.data(), sizeof(mine)) != 0) return bail(fail(TB_ERR_NCCL, "tp: the caller's all-gather failed"));
    for (int p = 0; p < size; ++p) {
      if (p == rank) { st->peer_block[p] = st->block; continue; }
      void* ptr = nullptr;
      e = cudaIpcOpenMemHandle(&ptr, all[p], cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) return bail(fail(TB_ERR_CUDA, "cudaIpcOpenMemHandle(rank %d): %s", p, cudaGetErrorString(e)));
      st->peer_block[p] = static_cast<char*>(ptr);
    }
    // nobody may start an exchange before every rank has mapped every block
    int token = 1;
    std::vector<int> tokens(size);
    if (allgather(user, &token, tokens.data(), sizeof(int)) != 0) return bail(fail(TB_ERR_NCCL, "tp: the caller's all-gather failed"));
    st->fused = true;
  }
  *out = st;
  return TB_OK;
}

}  // namespace tb

extern "C" tb_status tb_tp_unique_id(uint8_t id[128]) {
  if (!id) return tb::fail(TB_ERR_ARG, "tb_tp_unique_id: null buffer");
  tb::NcclApi* api = tb::nccl();
  if (!api) return tb::fail(TB_ERR_NCCL, "libnccl.so.2 could not be loaded: %s", dlerror());
  tb::NcclId nid;
  int r = api->get_unique_id(&nid);
  if (r != 0) return tb::fail(TB_ERR_NCCL, "ncclGetUniqueId failed: %s", api->err_string ? api->err_string(r) : "?");
  memcpy(id, nid.internal, 128);
  return TB_OK;
}
