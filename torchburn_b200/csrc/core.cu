// C ABI: error state, device report, the raw kernel surface and the
// QuantizedLinear handle.
#include <cstring>
#include <mutex>
#include <new>

#include "tb_common.cuh"
#include "tp.cuh"

namespace tb {

namespace {
unsigned long long* g_tl_base = nullptr;
int64_t g_tl_blocks = 0, g_tl_next = 0;
}  // namespace
void timeline_register(void* device_buffer, int64_t bytes) {
  g_tl_base = static_cast<unsigned long long*>(device_buffer);
  g_tl_blocks = device_buffer ? bytes / (int64_t)(kTlBlock * sizeof(unsigned long long)) : 0;
  g_tl_next = 0;
}
unsigned long long* timeline_next_block() {
  if (!g_tl_base || g_tl_next >= g_tl_blocks) return nullptr;
  return g_tl_base + (g_tl_next++) * kTlBlock;
}
int timeline_blocks_used() { return (int)g_tl_next; }


namespace {
thread_local char g_err[512] = "";
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

tb_status fail(tb_status code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  if (dev >= 0 && dev < 64) cached[dev] = n;
  return n;
}

// Copies `bytes` from host or device memory into a fresh device allocation.
tb_status upload(void** dst, const void* src, size_t bytes, tb_space space) {
  *dst = nullptr;
  if (bytes == 0) return TB_OK;
  TB_CUDA_TRY(cudaMalloc(dst, bytes));
  cudaError_t e = cudaMemcpy(*dst, src, bytes,
                             space == TB_HOST ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice);
  if (e != cudaSuccess) {
    cudaFree(*dst);
    *dst = nullptr;
    return fail(TB_ERR_CUDA, "weight upload failed: %s", cudaGetErrorString(e));
  }
  return TB_OK;
}

}  // namespace tb

using namespace tb;

struct tb_linear {
  uint8_t* qweight = nullptr;
  float* scales = nullptr;
  float* bias = nullptr;
  int64_t n = 0, k = 0;
  int g = 0;
  int device = 0;
  // pinned + device staging for host callers, grown on demand
  float *h_x = nullptr, *h_out = nullptr, *d_x = nullptr, *d_out = nullptr;
  int64_t stage_m = 0;
  std::mutex mu;
};

namespace {

tb_status ensure_stage(tb_linear* lin, int64_t m) {
  if (m <= lin->stage_m) return TB_OK;
  cudaFreeHost(lin->h_x); cudaFreeHost(lin->h_out); cudaFree(lin->d_x); cudaFree(lin->d_out);
  lin->h_x = lin->h_out = lin->d_x = lin->d_out = nullptr;
  lin->stage_m = 0;
  TB_CUDA_TRY(cudaMallocHost(&lin->h_x, sizeof(float) * m * lin->k));
  TB_CUDA_TRY(cudaMallocHost(&lin->h_out, sizeof(float) * m * lin->n));
  TB_CUDA_TRY(cudaMalloc(&lin->d_x, sizeof(float) * m * lin->k));
  TB_CUDA_TRY(cudaMalloc(&lin->d_out, sizeof(float) * m * lin->n));
  lin->stage_m = m;
  return TB_OK;
}

// Shape rules of w4a32_grouped_linear, src/quantization/packed_v2.rs:573-596.
tb_status check_linear_shape(int64_t n, int64_t k, int g) {
  if (n < 1 || k < 1) return fail(TB_ERR_SHAPE, "TB_UNSUPPORTED: w4a32_grouped_linear: empty weight [%lld, %lld]", (long long)n, (long long)k);
  if (g != 32 && g != 64 && g != 128) return fail(TB_ERR_SHAPE, "TB_UNSUPPORTED: group_size %d (supported: 32, 64, 128)", g);
  if (k % g != 0) return fail(TB_ERR_SHAPE, "TB_UNSUPPORTED: in_features %lld not a multiple of group_size %d", (long long)k, g);
  return TB_OK;
}

}  // namespace

extern "C" {

int32_t tb_abi_version(void) { return TB_ABI_VERSION; }

const char* tb_last_error_string(void) { return g_err; }

tb_status tb_device_report(char* buf, size_t cap) {
  if (!buf || cap == 0) return fail(TB_ERR_ARG, "tb_device_report: null buffer");
  int dev = 0;
  TB_CUDA_TRY(cudaGetDevice(&dev));
  cudaDeviceProp pr;
  TB_CUDA_TRY(cudaGetDeviceProperties(&pr, dev));
  int rt = 0, drv = 0;
  cudaRuntimeGetVersion(&rt);
  cudaDriverGetVersion(&drv);
  snprintf(buf, cap,
           "{\"device\": %d, \"name\": \"%s\", \"sm\": \"%d.%d\", \"sm_count\": %d, "
           "\"global_mem_bytes\": %zu, \"smem_per_block_optin\": %zu, \"l2_bytes\": %d, "
           "\"cuda_runtime\": %d, \"cuda_driver\": %d, \"built_for\": \"sm_100a\"}",
           dev, pr.name, pr.major, pr.minor, pr.multiProcessorCount, (size_t)pr.totalGlobalMem,
           (size_t)pr.sharedMemPerBlockOptin, pr.l2CacheSize, rt, drv);
  return TB_OK;
}

tb_status tb_gemv_w4a32_grouped(const float* x, const uint8_t* w, const float* scales,
                                const float* bias, float* out, int64_t n, int64_t k,
                                int32_t group_size, void* stream) {
  return tb_gemm_w4a32_grouped(x, w, scales, bias, out, 1, n, k, group_size, stream);
}

tb_status tb_gemm_w4a32_grouped(const float* x, const uint8_t* w, const float* scales,
                                const float* bias, float* out, int64_t m, int64_t n, int64_t k,
                                int32_t group_size, void* stream) {
  if (m == 0) return TB_OK;  // empty batch: nothing to do (the reference returns an empty tensor)
  GemvArgs a;
  a.x = x; a.w = w; a.scales = scales; a.bias = bias; a.out = out;
  a.m = (int)m; a.n = n; a.k = k; a.g = group_size;
  if (m < 0 || m > (1 << 20)) return fail(TB_ERR_SHAPE, "gemm: m=%lld out of range", (long long)m);
  return launch_w4_gemv(a, as_stream(stream));
}

tb_status tb_swiglu_gemv_w4a32(const float* x, const uint8_t* gate_w, const float* gate_s,
                               const float* gate_b, const uint8_t* up_w, const float* up_s,
                               const float* up_b, float* h, int64_t m, int64_t n, int64_t k,
                               int32_t group_size, void* stream) {
  if (m == 0) return TB_OK;
  if (!up_w || !up_s) return fail(TB_ERR_ARG, "swiglu: null up projection");
  GemvArgs a;
  a.x = x; a.w = gate_w; a.scales = gate_s; a.bias = gate_b;
  a.w2 = up_w; a.scales2 = up_s; a.bias2 = up_b;
  a.out = h; a.m = (int)m; a.n = n; a.k = k; a.g = group_size;
  if (m < 0 || m > (1 << 20)) return fail(TB_ERR_SHAPE, "swiglu: m=%lld out of range", (long long)m);
  return launch_w4_gemv(a, as_stream(stream));
}

tb_status tb_fast_rms_norm(const float* x, const float* w, float* out, int64_t m, int64_t n,
                           float eps, void* stream) {
  return launch_rms_norm(x, w, out, m, n, eps, as_stream(stream));
}

tb_status tb_quantize_weight_int4_grouped(const float* w, int64_t n, int64_t k,
                                          int32_t group_size, uint8_t* packed, float* scales,
                                          void* stream) {
  return launch_quantize_int4(w, n, k, group_size, packed, scales, as_stream(stream));
}

size_t tb_attention_scratch_bytes(int32_t batch, int32_t num_heads, int32_t num_kv_heads,
                                  int32_t head_dim, int64_t max_seq_len) {
  if (batch < 1 || num_heads < 1 || num_kv_heads < 1 || head_dim < 1 || max_seq_len < 1) return 0;
  return attention_scratch_bytes(batch, num_heads, num_kv_heads, head_dim, max_seq_len);
}

tb_status tb_attention_decode(const float* qkv, float* k_cache, float* v_cache,
                              const float* cos_table, const float* sin_table,
                              const int32_t* offsets, float* out, void* scratch, int32_t batch,
                              int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
                              int64_t max_seq_len, void* stream) {
  AttnArgs a;
  a.qkv = qkv; a.k_cache = k_cache; a.v_cache = v_cache; a.cos_t = cos_table; a.sin_t = sin_table;
  a.offsets = offsets; a.out = out; a.scratch = scratch; a.batch = batch; a.num_heads = num_heads;
  a.num_kv_heads = num_kv_heads; a.head_dim = head_dim; a.max_seq_len = max_seq_len;
  return launch_attention_decode(a, as_stream(stream));
}

size_t tb_attention_static_scratch_bytes(void) { return static_attention_scratch_capacity(); }

tb_status tb_attention_decode_static(const float* qkv, float* k_cache, float* v_cache,
                                     const float* cos_table, const float* sin_table,
                                     const int32_t* offsets, float* out, int32_t batch,
                                     int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
                                     int64_t max_seq_len, void* stream) {
  if (batch < 1 || num_heads < 1 || num_kv_heads < 1 || head_dim < 1 || max_seq_len < 1)
    return fail(TB_ERR_SHAPE, "tb_attention_decode_static: empty shape");
  const size_t need = attention_scratch_bytes(batch, num_heads, num_kv_heads, head_dim, max_seq_len);
  if (need > static_attention_scratch_capacity())
    return fail(TB_ERR_UNSUPPORTED,
                "tb_attention_decode_static: this shape needs %zu bytes of scratch, the built-in block holds %zu; "
                "use tb_attention_decode with caller-provided scratch",
                need, static_attention_scratch_capacity());
  void* scratch = nullptr;
  TB_TRY(static_attention_scratch(&scratch));
  // The block keeps whatever the previous call (possibly of another shape) left behind:
  // the ticket counters and the error word of this shape must start at zero.
  size_t cbytes = 0;
  const size_t coff = attention_counters_offset(batch, num_heads, num_kv_heads, head_dim, max_seq_len, &cbytes);
  TB_CUDA_TRY(cudaMemsetAsync(static_cast<char*>(scratch) + coff, 0, cbytes, as_stream(stream)));
  AttnArgs a;
  a.qkv = qkv; a.k_cache = k_cache; a.v_cache = v_cache; a.cos_t = cos_table; a.sin_t = sin_table;
  a.offsets = offsets; a.out = out; a.scratch = scratch; a.batch = batch; a.num_heads = num_heads;
  a.num_kv_heads = num_kv_heads; a.head_dim = head_dim; a.max_seq_len = max_seq_len;
  return launch_attention_decode(a, as_stream(stream));
}

void tb_set_attention_chunk(int32_t tc) { set_attention_chunk_override(tc); }
void tb_set_attention_tuning(int32_t ctas_per_sm, int32_t ring_stages) {
  set_attention_tuning(ctas_per_sm < 0 ? 0 : ctas_per_sm, ring_stages < 0 ? 0 : ring_stages);
}

void tb_set_gemv_tuning(int32_t xmode, int32_t rows_per_warp, int32_t warps) { set_gemv_tuning(xmode, rows_per_warp, warps); }

void tb_release_workspaces(void) { release_workspaces(); }

void tb_set_stream_tuning(int32_t enabled, int32_t ctas_per_sm, int32_t ring_kb, int32_t epl, int32_t groups) {
  set_stream_tuning(enabled, ctas_per_sm, ring_kb, epl, groups);
}

void tb_debug_timeline(void* device_buffer, int64_t bytes) { timeline_register(device_buffer, bytes); }
void tb_debug_step_flags(int32_t flags) { set_step_debug(flags); }
tb_status tb_debug_wait_probe(int64_t limit_cycles) { return step_wait_probe((long long)limit_cycles); }
void tb_debug_step_wait_limit(int64_t cycles) {
  set_step_wait_limit((long long)cycles);
  tp_set_wait_limit((long long)cycles);
}

tb_status tb_debug_step_gemv(const float* x, const uint8_t* w, const float* scales, const float* bias, const uint8_t* w2,
                             const float* scales2, float* out, int64_t n, int64_t k, int32_t group_size, void* stream) {
  GemvArgs a;
  a.x = x; a.w = w; a.scales = scales; a.bias = bias; a.w2 = w2; a.scales2 = scales2; a.out = out;
  a.m = 1; a.n = n; a.k = k; a.g = group_size;
  return launch_w4_step_gemv(a, as_stream(stream));
}
int32_t tb_debug_timeline_blocks(void) { return timeline_blocks_used(); }

int32_t tb_device_fault_flag(void) {
  const int a = stream_fault_flag(), b = attention_fault_flag(), c = step_fault_flag(), e = tc5_fault_flag();
  if (a < 0 || b < 0 || c < 0 || e < 0) return -1;
  return (a | b | c | e) ? 1 : 0;
}

/* ------------------------------------------------------------ QuantizedLinear */

tb_status tb_linear_create(tb_linear** out, const uint8_t* qweight, const float* scales,
                           const float* bias, int64_t out_features, int64_t in_features,
                           int32_t group_size, tb_space weight_space) {
  if (!out) return fail(TB_ERR_ARG, "tb_linear_create: null out");
  *out = nullptr;
  if (!qweight || !scales) return fail(TB_ERR_ARG, "tb_linear_create: null weight");
  TB_TRY(check_linear_shape(out_features, in_features, group_size));
  tb_linear* lin = new (std::nothrow) tb_linear();
  if (!lin) return fail(TB_ERR_OOM, "tb_linear_create: host allocation failed");
  lin->n = out_features; lin->k = in_features; lin->g = group_size;
  cudaGetDevice(&lin->device);
  tb_status s = upload((void**)&lin->qweight, qweight, (size_t)out_features * (in_features / 2), weight_space);
  if (s == TB_OK) s = upload((void**)&lin->scales, scales, sizeof(float) * out_features * (in_features / group_size), weight_space);
  if (s == TB_OK && bias) s = upload((void**)&lin->bias, bias, sizeof(float) * out_features, weight_space);
  if (s != TB_OK) {
    tb_linear_destroy(lin);
    return s;
  }
  *out = lin;
  return TB_OK;
}

void tb_linear_destroy(tb_linear* lin) {
  if (!lin) return;
  cudaFree(lin->qweight); cudaFree(lin->scales); cudaFree(lin->bias);
  cudaFreeHost(lin->h_x); cudaFreeHost(lin->h_out); cudaFree(lin->d_x); cudaFree(lin->d_out);
  delete lin;
}

tb_status tb_linear_device_ptrs(const tb_linear* lin, const uint8_t** qweight, const float** scales,
                                const float** bias) {
  if (!lin) return fail(TB_ERR_ARG, "tb_linear_device_ptrs: null handle");
  if (qweight) *qweight = lin->qweight;
  if (scales) *scales = lin->scales;
  if (bias) *bias = lin->bias;
  return TB_OK;
}

tb_status tb_linear_forward(tb_linear* lin, const float* x, int64_t m, float* out,
                            tb_space io_space, void* stream) {
  if (!lin) return fail(TB_ERR_ARG, "tb_linear_forward: null handle");
  if (m == 0) return TB_OK;
  if (!x || !out) return fail(TB_ERR_ARG, "tb_linear_forward: null x/out");
  if (m < 0) return fail(TB_ERR_SHAPE, "tb_linear_forward: m=%lld", (long long)m);
  cudaStream_t st = as_stream(stream);
  if (io_space == TB_DEVICE)
    return tb_gemm_w4a32_grouped(x, lin->qweight, lin->scales, lin->bias, out, m, lin->n, lin->k, lin->g, stream);
  std::lock_guard<std::mutex> lock(lin->mu);
  TB_TRY(ensure_stage(lin, m));
  memcpy(lin->h_x, x, sizeof(float) * m * lin->k);
  TB_CUDA_TRY(cudaMemcpyAsync(lin->d_x, lin->h_x, sizeof(float) * m * lin->k, cudaMemcpyHostToDevice, st));
  TB_TRY(tb_gemm_w4a32_grouped(lin->d_x, lin->qweight, lin->scales, lin->bias, lin->d_out, m, lin->n, lin->k, lin->g, stream));
  TB_CUDA_TRY(cudaMemcpyAsync(lin->h_out, lin->d_out, sizeof(float) * m * lin->n, cudaMemcpyDeviceToHost, st));
  TB_CUDA_TRY(cudaStreamSynchronize(st));
  memcpy(out, lin->h_out, sizeof(float) * m * lin->n);
  return TB_OK;
}

tb_status tb_fused_swiglu_mlp(tb_linear* gate, tb_linear* up, tb_linear* down, const float* x,
                              int64_t m, float* out, tb_space io_space, void* stream) {
  if (!gate || !up || !down) return fail(TB_ERR_ARG, "tb_fused_swiglu_mlp: null handle");
  if (m == 0) return TB_OK;
  if (!x || !out || m < 0) return fail(TB_ERR_ARG, "tb_fused_swiglu_mlp: bad x/out/m");
  if (gate->k != up->k || gate->n != up->n || down->k != gate->n || gate->g != up->g || gate->g != down->g)
    return fail(TB_ERR_SHAPE, "TB_UNSUPPORTED: fused_swiglu_mlp: gate [%lld,%lld] up [%lld,%lld] down [%lld,%lld] do not chain",
                (long long)gate->n, (long long)gate->k, (long long)up->n, (long long)up->k, (long long)down->n, (long long)down->k);
  cudaStream_t st = as_stream(stream);
  const int64_t H = gate->k, I = gate->n, O = down->n;
  float *d_x = nullptr, *d_h = nullptr, *d_o = nullptr;
  tb_status s = TB_OK;
  auto cleanup = [&]() { if (io_space == TB_HOST) { cudaFree(d_x); cudaFree(d_o); } cudaFree(d_h); };
  cudaError_t e = cudaMalloc(&d_h, sizeof(float) * m * I);
  if (e != cudaSuccess) return fail(TB_ERR_OOM, "fused_swiglu_mlp: %s", cudaGetErrorString(e));
  if (io_space == TB_HOST) {
    if (cudaMalloc(&d_x, sizeof(float) * m * H) != cudaSuccess || cudaMalloc(&d_o, sizeof(float) * m * O) != cudaSuccess) {
      cleanup();
      return fail(TB_ERR_OOM, "fused_swiglu_mlp: device staging allocation failed");
    }
    e = cudaMemcpyAsync(d_x, x, sizeof(float) * m * H, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) { cleanup(); return fail(TB_ERR_CUDA, "fused_swiglu_mlp: %s", cudaGetErrorString(e)); }
  } else {
    d_x = const_cast<float*>(x);
    d_o = out;
  }
  s = tb_swiglu_gemv_w4a32(d_x, gate->qweight, gate->scales, gate->bias, up->qweight, up->scales, up->bias, d_h, m, I, H, gate->g, stream);
  if (s == TB_OK) s = tb_gemm_w4a32_grouped(d_h, down->qweight, down->scales, down->bias, d_o, m, O, I, down->g, stream);
  if (s == TB_OK && io_space == TB_HOST) {
    e = cudaMemcpyAsync(out, d_o, sizeof(float) * m * O, cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) s = fail(TB_ERR_CUDA, "fused_swiglu_mlp: %s", cudaGetErrorString(e));
  }
  e = cudaStreamSynchronize(st);
  if (s == TB_OK && e != cudaSuccess) s = fail(TB_ERR_CUDA, "fused_swiglu_mlp: %s", cudaGetErrorString(e));
  cleanup();
  return s;
}

tb_status tb_fused_attention_step(tb_linear* qkv, tb_linear* o, const float* x, float* k_cache,
                                  float* v_cache, const float* cos_p, const float* sin_p,
                                  int64_t offset, int32_t num_heads, int32_t num_kv_heads,
                                  int32_t head_dim, int64_t max_seq_len, float* out,
                                  tb_space io_space, void* stream) {
  if (!qkv || !o || !x || !k_cache || !v_cache || !cos_p || !sin_p || !out)
    return fail(TB_ERR_ARG, "tb_fused_attention_step: null argument");
  const int64_t H = qkv->k, q_dim = (int64_t)num_heads * head_dim;
  const int64_t total = q_dim + 2ll * num_kv_heads * head_dim;
  if (qkv->n != total || o->k != q_dim)
    return fail(TB_ERR_SHAPE, "TB_UNSUPPORTED: fused_attention_step: qkv rows %lld != %lld or o in_features %lld != %lld",
                (long long)qkv->n, (long long)total, (long long)o->k, (long long)q_dim);
  if (offset < 0 || offset >= max_seq_len)
    return fail(TB_ERR_ARG, "fused_attention_step: offset %lld outside the cache (max_seq_len %lld)", (long long)offset, (long long)max_seq_len);
  cudaStream_t st = as_stream(stream);
  const size_t sbytes = attention_scratch_bytes(1, num_heads, num_kv_heads, head_dim, max_seq_len);
  // one device block: x | cos | sin | qkv | attn | out | offset | scratch
  const size_t fl = (size_t)H + 2 * head_dim + total + q_dim + o->n;
  const size_t hdr = ((fl * sizeof(float) + sizeof(int32_t)) + 255) & ~(size_t)255;
  char* blk = nullptr;
  cudaError_t e = cudaMalloc(&blk, hdr + sbytes);
  if (e != cudaSuccess) return fail(TB_ERR_OOM, "fused_attention_step: %s", cudaGetErrorString(e));
  float* d_x = reinterpret_cast<float*>(blk);
  float* d_cos = d_x + H;
  float* d_sin = d_cos + head_dim;
  float* d_qkv = d_sin + head_dim;
  float* d_attn = d_qkv + total;
  float* d_out = d_attn + q_dim;
  int32_t* d_off = reinterpret_cast<int32_t*>(d_out + o->n);
  tb_status s = TB_OK;
  const cudaMemcpyKind kin = io_space == TB_HOST ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
  const int32_t off32 = (int32_t)offset;
  auto chk = [&](cudaError_t err) { if (err != cudaSuccess && s == TB_OK) s = fail(TB_ERR_CUDA, "fused_attention_step: %s", cudaGetErrorString(err)); };
  chk(cudaMemsetAsync(blk + hdr, 0, sbytes, st));
  chk(cudaMemcpyAsync(d_x, x, sizeof(float) * H, kin, st));
  chk(cudaMemcpyAsync(d_cos, cos_p, sizeof(float) * head_dim, kin, st));
  chk(cudaMemcpyAsync(d_sin, sin_p, sizeof(float) * head_dim, kin, st));
  chk(cudaMemcpyAsync(d_off, &off32, sizeof(int32_t), cudaMemcpyHostToDevice, st));
  if (s == TB_OK) s = tb_gemm_w4a32_grouped(d_x, qkv->qweight, qkv->scales, qkv->bias, d_qkv, 1, total, H, qkv->g, stream);
  if (s == TB_OK) {
    AttnArgs a;
    a.qkv = d_qkv; a.k_cache = k_cache; a.v_cache = v_cache; a.cos_t = d_cos; a.sin_t = d_sin;
    a.offsets = d_off; a.out = d_attn; a.scratch = blk + hdr; a.batch = 1; a.num_heads = num_heads;
    a.num_kv_heads = num_kv_heads; a.head_dim = head_dim; a.max_seq_len = max_seq_len;
    a.per_call_tables = true;
    s = launch_attention_decode(a, st);
  }
  if (s == TB_OK) s = tb_gemm_w4a32_grouped(d_attn, o->qweight, o->scales, o->bias, d_out, 1, o->n, q_dim, o->g, stream);
  if (s == TB_OK)
    chk(cudaMemcpyAsync(out, d_out, sizeof(float) * o->n, io_space == TB_HOST ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice, st));
  chk(cudaStreamSynchronize(st));
  cudaFree(blk);
  return s;
}

/* fused_transformer_layer_step_w4a32: steps 1-10 of one layer, in place on x. */
tb_status tb_fused_transformer_layer_step(float* x, const tb_layer_step_weights* w, float* k_cache, float* v_cache,
                                          const float* cos_p, const float* sin_p, int64_t offset, int64_t hidden_size,
                                          int64_t intermediate_size, int32_t num_heads, int32_t num_kv_heads,
                                          int32_t head_dim, int64_t max_seq_len, int32_t group_size, float eps,
                                          tb_space io_space, void* stream) {
  if (!x || !w || !k_cache || !v_cache || !cos_p || !sin_p) return fail(TB_ERR_ARG, "tb_fused_transformer_layer_step: null argument");
  if (!w->input_norm_w || !w->qkv_w || !w->qkv_s || !w->o_w || !w->o_s || !w->post_norm_w || !w->gate_w || !w->gate_s ||
      !w->up_w || !w->up_s || !w->down_w || !w->down_s)
    return fail(TB_ERR_ARG, "tb_fused_transformer_layer_step: a weight tensor is missing");
  if (num_heads < 1 || num_kv_heads < 1 || head_dim < 2 || hidden_size < 1 || intermediate_size < 1)
    return fail(TB_ERR_SHAPE, "TB_UNSUPPORTED: fused_transformer_layer_step: empty shape");
  const int64_t H = hidden_size, I = intermediate_size, q_dim = (int64_t)num_heads * head_dim;
  const int64_t total = q_dim + 2ll * num_kv_heads * head_dim;
  TB_TRY(check_linear_shape(total, H, group_size));
  TB_TRY(check_linear_shape(H, q_dim, group_size));
  TB_TRY(check_linear_shape(I, H, group_size));
  TB_TRY(check_linear_shape(H, I, group_size));
  if (offset < 0 || offset >= max_seq_len)
    return fail(TB_ERR_ARG, "fused_transformer_layer_step: offset %lld outside the cache (max_seq_len %lld)", (long long)offset, (long long)max_seq_len);
  cudaStream_t st = as_stream(stream);
  const size_t sbytes = attention_scratch_bytes(1, num_heads, num_kv_heads, head_dim, max_seq_len);
  // one device block: x | cos | sin | qkv | attn | h | offset | attention scratch
  const size_t fl = (size_t)H + 2 * head_dim + total + q_dim + I;
  const size_t hdr = ((fl * sizeof(float) + sizeof(int32_t)) + 255) & ~(size_t)255;
  char* blk = nullptr;
  cudaError_t e = cudaMalloc(&blk, hdr + sbytes);
  if (e != cudaSuccess) return fail(TB_ERR_OOM, "fused_transformer_layer_step: %s", cudaGetErrorString(e));
  float* d_x = reinterpret_cast<float*>(blk);
  float* d_cos = d_x + H;
  float* d_sin = d_cos + head_dim;
  float* d_qkv = d_sin + head_dim;
  float* d_attn = d_qkv + total;
  float* d_h = d_attn + q_dim;
  int32_t* d_off = reinterpret_cast<int32_t*>(d_h + I);
  tb_status s = TB_OK;
  const cudaMemcpyKind kin = io_space == TB_HOST ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
  const int32_t off32 = (int32_t)offset;
  auto chk = [&](cudaError_t err) { if (err != cudaSuccess && s == TB_OK) s = fail(TB_ERR_CUDA, "fused_transformer_layer_step: %s", cudaGetErrorString(err)); };
  chk(cudaMemsetAsync(blk + hdr, 0, sbytes, st));
  chk(cudaMemcpyAsync(d_x, x, sizeof(float) * H, kin, st));
  chk(cudaMemcpyAsync(d_cos, cos_p, sizeof(float) * head_dim, kin, st));
  chk(cudaMemcpyAsync(d_sin, sin_p, sizeof(float) * head_dim, kin, st));
  chk(cudaMemcpyAsync(d_off, &off32, sizeof(int32_t), cudaMemcpyHostToDevice, st));
  if (s == TB_OK) {  // 1 + 2: RMSNorm fused into the QKV projection
    GemvArgs a;
    a.x = d_x; a.w = w->qkv_w; a.scales = w->qkv_s; a.bias = w->qkv_b; a.norm_w = w->input_norm_w; a.eps = eps;
    a.out = d_qkv; a.m = 1; a.n = total; a.k = H; a.g = group_size;
    s = launch_w4_gemv(a, st);
  }
  if (s == TB_OK) {  // 3 + 4 + 5: RoPE, cache write, attention
    AttnArgs a;
    a.qkv = d_qkv; a.k_cache = k_cache; a.v_cache = v_cache; a.cos_t = d_cos; a.sin_t = d_sin;
    a.offsets = d_off; a.out = d_attn; a.scratch = blk + hdr; a.batch = 1; a.num_heads = num_heads;
    a.num_kv_heads = num_kv_heads; a.head_dim = head_dim; a.max_seq_len = max_seq_len;
    a.per_call_tables = true;
    s = launch_attention_decode(a, st);
  }
  if (s == TB_OK) {  // 6 + 7: O projection, x += o_out
    GemvArgs a;
    a.x = d_attn; a.w = w->o_w; a.scales = w->o_s; a.bias = w->o_b; a.resid = d_x; a.out = d_x;
    a.m = 1; a.n = H; a.k = q_dim; a.g = group_size;
    s = launch_w4_gemv(a, st);
  }
  if (s == TB_OK) {  // 8 + 9a: RMSNorm fused into gate/up with the SwiGLU epilogue
    GemvArgs a;
    a.x = d_x; a.w = w->gate_w; a.scales = w->gate_s; a.bias = w->gate_b; a.w2 = w->up_w; a.scales2 = w->up_s; a.bias2 = w->up_b;
    a.norm_w = w->post_norm_w; a.eps = eps; a.out = d_h; a.m = 1; a.n = I; a.k = H; a.g = group_size;
    s = launch_w4_gemv(a, st);
  }
  if (s == TB_OK) {  // 9b + 10: down projection, x += mlp_out
    GemvArgs a;
    a.x = d_h; a.w = w->down_w; a.scales = w->down_s; a.bias = w->down_b; a.resid = d_x; a.out = d_x;
    a.m = 1; a.n = H; a.k = I; a.g = group_size;
    s = launch_w4_gemv(a, st);
  }
  if (s == TB_OK)
    chk(cudaMemcpyAsync(x, d_x, sizeof(float) * H, io_space == TB_HOST ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice, st));
  chk(cudaStreamSynchronize(st));
  cudaFree(blk);
  return s;
}

}  // extern "C"
