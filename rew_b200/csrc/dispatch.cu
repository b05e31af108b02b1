// Tier A: the EagerBackend proc slot of rew (src/rew/dispatch.nim:47-85) as a C
// call.  Every primitive the decoder layers dispatch (src/rew/ops/*.nim) maps to
// one kernel launch here instead of a compiled single-op StableHLO module
// (src/rew/eager.nim:1717-1767).  Attribute strings use rew's wire format
// (src/rew/eager.nim:934-948): integer lists as "[1,2]" or "@[1, 2]".
// Output shape / dtype rules follow src/rew/eager.nim:1061-1283.
#include <math.h>

#include <cstring>
#include <map>
#include <string>

#include "common.cuh"
#include "ptx.cuh"

using namespace rewb;

namespace rewb {
int moe_route_launch(Ctx* c, const float* logits, int64_t N, int E, int k, float* topw, int* topi);

namespace {

struct Strided {
  int nd;
  int64_t dims[8];      // iteration space
  int64_t in_str[8];    // element strides into the source
  int64_t out_str[8];   // element strides into the destination
  int64_t in_off, out_off;
};

template <typename T>
__global__ void strided_copy_kernel(const T* __restrict__ in, T* __restrict__ out, Strided s, int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  int64_t rem = i, io = s.in_off, oo = s.out_off;
#pragma unroll
  for (int d = 7; d >= 0; --d) {
    if (d < s.nd) {
      const int64_t c = rem % s.dims[d];
      rem /= s.dims[d];
      io += c * s.in_str[d];
      oo += c * s.out_str[d];
    }
  }
  out[oo] = in[io];
}

template <typename T> __device__ __forceinline__ float ld(const T* p, int64_t i);
template <> __device__ __forceinline__ float ld<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float ld<bf16>(const bf16* p, int64_t i) { return __bfloat162float(p[i]); }
template <> __device__ __forceinline__ float ld<int>(const int* p, int64_t i) { return (float)p[i]; }
template <typename T> __device__ __forceinline__ void st(T* p, int64_t i, float v);
template <> __device__ __forceinline__ void st<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void st<bf16>(bf16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

enum BinOp { B_ADD, B_SUB, B_MUL, B_DIV, B_MAX, B_MIN };
enum UnOp { U_NEG, U_EXP, U_SQRT, U_RSQRT, U_LOGISTIC, U_TANH, U_LOG };
enum CmpOp { C_LT, C_LE, C_GT, C_GE, C_EQ, C_NE };

template <typename T>
__global__ void binary_kernel(const T* a, const T* b, T* out, int64_t n, int op) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float x = ld<T>(a, i), y = ld<T>(b, i);
  float r;
  switch (op) {
    case B_ADD: r = x + y; break;
    case B_SUB: r = x - y; break;
    case B_MUL: r = x * y; break;
    case B_DIV: r = x / y; break;
    case B_MAX: r = fmaxf(x, y); break;
    default: r = fminf(x, y); break;
  }
  st<T>(out, i, r);
}
__global__ void binary_i32_kernel(const int* a, const int* b, int* out, int64_t n, int op) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int x = a[i], y = b[i];
  int r;
  switch (op) {
    case B_ADD: r = x + y; break;
    case B_SUB: r = x - y; break;
    case B_MUL: r = x * y; break;
    case B_DIV: r = y ? x / y : 0; break;
    case B_MAX: r = max(x, y); break;
    default: r = min(x, y); break;
  }
  out[i] = r;
}
template <typename T>
__global__ void unary_kernel(const T* a, T* out, int64_t n, int op) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float x = ld<T>(a, i);
  float r;
  switch (op) {
    case U_NEG: r = -x; break;
    case U_EXP: r = expf(x); break;
    case U_SQRT: r = sqrtf(x); break;
    case U_RSQRT: r = 1.0f / sqrtf(x); break;
    case U_LOGISTIC: r = 1.0f / (1.0f + expf(-x)); break;
    case U_TANH: r = tanhf(x); break;
    default: r = logf(x); break;
  }
  st<T>(out, i, r);
}
template <typename T>
__global__ void compare_kernel(const T* a, const T* b, uint8_t* out, int64_t n, int op) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const T x = a[i], y = b[i];
  bool r;
  switch (op) {
    case C_LT: r = x < y; break;
    case C_LE: r = x <= y; break;
    case C_GT: r = x > y; break;
    case C_GE: r = x >= y; break;
    case C_EQ: r = x == y; break;
    default: r = x != y; break;
  }
  out[i] = r ? 1 : 0;
}
template <typename T>
__global__ void select_kernel(const uint8_t* p, const T* a, const T* b, T* out, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = p[i] ? a[i] : b[i];
}
template <typename T>
__global__ void iota_kernel(T* out, int64_t n, int64_t inner, int64_t extent) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = (T)((i / inner) % extent);
}
// astype through double keeps int32 exact.
template <typename TS, typename TD>
__global__ void convert_kernel(const TS* in, TD* out, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = (TD)in[i];
}
__global__ void f32_to_bf16_kernel(const float* in, bf16* out, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16_rn(in[i]);
}
__global__ void bf16_to_f32_kernel(const bf16* in, float* out, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __bfloat162float(in[i]);
}

// One CTA per output element: reduce `len` contiguous values.
__global__ void __launch_bounds__(128) reduce_rows_kernel(const float* in, float* out, int64_t len, int is_max) {
  __shared__ float red[4];
  const float* r = in + (int64_t)blockIdx.x * len;
  float acc = is_max ? -INFINITY : 0.f;
  for (int64_t i = threadIdx.x; i < len; i += blockDim.x) acc = is_max ? fmaxf(acc, r[i]) : acc + r[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float v = __shfl_xor_sync(0xffffffffu, acc, o);
    acc = is_max ? fmaxf(acc, v) : acc + v;
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = red[0];
    for (int w = 1; w < 4; ++w) t = is_max ? fmaxf(t, red[w]) : t + red[w];
    out[blockIdx.x] = t;
  }
}

// Top-k of each row in descending order, ties towards the lower index
// (src/rew/ops/sort.nim:36-90 sorts the whole row twice; this selects k times).
__global__ void __launch_bounds__(256) topk_rows_kernel(const float* in, int64_t n, int k, float* vals, int* idx) {
  __shared__ float sv[8];
  __shared__ int si[8];
  __shared__ float pv_s;
  __shared__ int pi_s;
  const float* r = in + (int64_t)blockIdx.x * n;
  float pv = INFINITY;
  int pi = -1;
  for (int j = 0; j < k; ++j) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
      const float v = r[i];
      const bool after = (v < pv) || (v == pv && (int)i > pi);  // strictly later in (value desc, index asc) order
      if (after && (v > bv || (v == bv && (int)i < bi))) {
        bv = v;
        bi = (int)i;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if ((threadIdx.x & 31) == 0) {
      sv[threadIdx.x >> 5] = bv;
      si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < 8; ++w)
        if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) {
          bv = sv[w];
          bi = si[w];
        }
      vals[(int64_t)blockIdx.x * k + j] = bv;
      idx[(int64_t)blockIdx.x * k + j] = bi;
      pv_s = bv;
      pi_s = bi;
    }
    __syncthreads();
    pv = pv_s;
    pi = pi_s;
  }
}

// ---------------------------------------------------------------- host helpers
typedef std::map<std::string, std::string> Attrs;

bool parse_ints(const std::string& s, std::vector<int64_t>* out) {
  out->clear();
  size_t i = 0;
  while (i < s.size()) {
    const char ch = s[i];
    if (ch == '-' || (ch >= '0' && ch <= '9')) {
      size_t j = i + 1;
      while (j < s.size() && s[j] >= '0' && s[j] <= '9') ++j;
      out->push_back(std::stoll(s.substr(i, j - i)));
      i = j;
    } else if (ch == '[' || ch == ']' || ch == '@' || ch == ',' || ch == ' ') {
      ++i;
    } else {
      return false;
    }
  }
  return true;
}

int get_ints(const Attrs& a, const char* op, const char* key, std::vector<int64_t>* out) {
  auto it = a.find(key);
  RB_REQUIRE(it != a.end(), std::string(op) + ": missing attribute '" + key + "'");
  RB_REQUIRE(parse_ints(it->second, out), std::string(op) + ": attribute '" + key + "' is not an integer list: " + it->second);
  return REWB200_OK;
}

int dtype_from_name(const std::string& n) {
  if (n == "float32" || n == "dtFloat32" || n == "f32") return REWB200_F32;
  if (n == "bfloat16" || n == "dtBFloat16" || n == "bf16") return REWB200_BF16;
  if (n == "int32" || n == "dtInt32" || n == "i32") return REWB200_I32;
  if (n == "int64" || n == "dtInt64" || n == "i64") return REWB200_I64;
  if (n == "bool" || n == "dtBool") return REWB200_BOOL;
  if (n == "uint8" || n == "dtUint8") return REWB200_U8;
  return -1;
}

void contiguous_strides(const int64_t* dims, int nd, int64_t* str) {
  int64_t s = 1;
  for (int i = nd - 1; i >= 0; --i) {
    str[i] = s;
    s *= dims[i];
  }
}

int run_strided(Ctx* c, const void* in, void* out, const Strided& s, size_t elem) {
  int64_t total = 1;
  for (int i = 0; i < s.nd; ++i) total *= s.dims[i];
  if (total == 0) return REWB200_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  switch (elem) {
    case 1: strided_copy_kernel<uint8_t><<<blocks, 256, 0, c->stream>>>((const uint8_t*)in, (uint8_t*)out, s, total); break;
    case 2: strided_copy_kernel<uint16_t><<<blocks, 256, 0, c->stream>>>((const uint16_t*)in, (uint16_t*)out, s, total); break;
    case 4: strided_copy_kernel<uint32_t><<<blocks, 256, 0, c->stream>>>((const uint32_t*)in, (uint32_t*)out, s, total); break;
    case 8: strided_copy_kernel<uint64_t><<<blocks, 256, 0, c->stream>>>((const uint64_t*)in, (uint64_t*)out, s, total); break;
    default: return fail("unsupported element size");
  }
  RB_CUDA(cudaGetLastError());
  ++g_launch_total;
  return REWB200_OK;
}

#define LAUNCH1D(kernel, n, ...)                                                        \
  do {                                                                                  \
    if ((n) > 0) {                                                                      \
      kernel<<<(unsigned)(((n) + 255) / 256), 256, 0, c->stream>>>(__VA_ARGS__);        \
      RB_CUDA(cudaGetLastError());                                                      \
      ++g_launch_total;                                                                 \
    }                                                                                   \
  } while (0)

bool same_shape(const rewb200_buffer* a, const rewb200_buffer* b) {
  if (a->ndims != b->ndims) return false;
  for (int i = 0; i < a->ndims; ++i)
    if (a->dims[i] != b->dims[i]) return false;
  return true;
}

std::string shape_str(const rewb200_buffer* b) {
  std::string s = "[";
  for (int i = 0; i < b->ndims; ++i) s += (i ? "," : "") + std::to_string(b->dims[i]);
  return s + "]";
}

int op_binary(Ctx* c, const char* op, int code, rewb200_buffer* const* x, rewb200_buffer** out) {
  RB_REQUIRE(same_shape(x[0], x[1]), std::string(op) + ": shape mismatch " + shape_str(x[0]) + " vs " + shape_str(x[1]));
  RB_REQUIRE(x[0]->dtype == x[1]->dtype, std::string(op) + ": dtype mismatch");
  RB_TRY(buffer_new(c, x[0]->dtype, x[0]->dims, x[0]->ndims, out));
  const int64_t n = x[0]->numel();
  if (x[0]->dtype == REWB200_F32) LAUNCH1D(binary_kernel<float>, n, (const float*)x[0]->ptr, (const float*)x[1]->ptr, (float*)(*out)->ptr, n, code);
  else if (x[0]->dtype == REWB200_BF16) LAUNCH1D(binary_kernel<bf16>, n, (const bf16*)x[0]->ptr, (const bf16*)x[1]->ptr, (bf16*)(*out)->ptr, n, code);
  else if (x[0]->dtype == REWB200_I32) LAUNCH1D(binary_i32_kernel, n, (const int*)x[0]->ptr, (const int*)x[1]->ptr, (int*)(*out)->ptr, n, code);
  else return fail(std::string(op) + ": dtype must be float32, bfloat16 or int32");
  return REWB200_OK;
}

int op_unary(Ctx* c, const char* op, int code, rewb200_buffer* const* x, rewb200_buffer** out) {
  RB_TRY(buffer_new(c, x[0]->dtype, x[0]->dims, x[0]->ndims, out));
  const int64_t n = x[0]->numel();
  if (x[0]->dtype == REWB200_F32) LAUNCH1D(unary_kernel<float>, n, (const float*)x[0]->ptr, (float*)(*out)->ptr, n, code);
  else if (x[0]->dtype == REWB200_BF16) LAUNCH1D(unary_kernel<bf16>, n, (const bf16*)x[0]->ptr, (bf16*)(*out)->ptr, n, code);
  else return fail(std::string(op) + ": dtype must be float32 or bfloat16");
  return REWB200_OK;
}

int op_transpose(Ctx* c, const rewb200_buffer* x, const std::vector<int64_t>& perm, rewb200_buffer** out) {
  RB_REQUIRE((int)perm.size() == x->ndims, "transpose: permutation rank mismatch");
  int64_t istr[8], od[8];
  contiguous_strides(x->dims, x->ndims, istr);
  Strided s;
  memset(&s, 0, sizeof(s));
  s.nd = x->ndims;
  std::vector<bool> seen(x->ndims, false);
  for (int i = 0; i < x->ndims; ++i) {
    RB_REQUIRE(perm[i] >= 0 && perm[i] < x->ndims && !seen[perm[i]], "transpose: invalid permutation");
    seen[perm[i]] = true;
    od[i] = x->dims[perm[i]];
    s.dims[i] = od[i];
    s.in_str[i] = istr[perm[i]];
  }
  contiguous_strides(od, x->ndims, s.out_str);
  RB_TRY(buffer_new(c, x->dtype, od, x->ndims, out));
  return run_strided(c, x->ptr, (*out)->ptr, s, dtype_size(x->dtype));
}

}  // namespace
}  // namespace rewb

extern "C" int rewb200_dispatch(const char* op_c, rewb200_buffer* const* x, int n_operands, const char* const* attr_keys,
                                const char* const* attr_vals, int n_attrs, rewb200_buffer** out, int* n_out) {
  RB_REQUIRE(op_c && out && n_out && *n_out >= 1, "dispatchEager: NULL argument");
  const std::string op(op_c);
  Attrs at;
  for (int i = 0; i < n_attrs; ++i) at[attr_keys[i]] = attr_vals[i] ? attr_vals[i] : "";
  for (int i = 0; i < n_operands; ++i) RB_REQUIRE(x[i] != nullptr, "eager op '" + op + "': NULL operand");
  for (int i = 1; i < n_operands; ++i)
    RB_REQUIRE(x[i]->slot == x[0]->slot, "eager op '" + op + "': cross-device operands forbidden");
  Ctx* c = ctx_get(n_operands ? x[0]->slot : 0);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  const int cap = *n_out;
  *n_out = 1;
  auto need = [&](int n) -> int {
    RB_REQUIRE(n_operands == n, "eager op '" + op + "': expected " + std::to_string(n) + " operands, got " + std::to_string(n_operands));
    return REWB200_OK;
  };

  static const std::map<std::string, int> bin = {{"add", B_ADD}, {"sub", B_SUB}, {"mul", B_MUL}, {"divide", B_DIV},
                                                 {"maximum", B_MAX}, {"minimum", B_MIN}};
  static const std::map<std::string, int> un = {{"neg", U_NEG}, {"exp", U_EXP}, {"sqrt", U_SQRT}, {"rsqrt", U_RSQRT},
                                                {"logistic", U_LOGISTIC}, {"tanh", U_TANH}, {"log", U_LOG}};
  if (bin.count(op)) {
    RB_TRY(need(2));
    return op_binary(c, op_c, bin.at(op), x, out);
  }
  if (un.count(op)) {
    RB_TRY(need(1));
    return op_unary(c, op_c, un.at(op), x, out);
  }
  if (op == "reshape") {
    RB_TRY(need(1));
    std::vector<int64_t> shp;
    RB_TRY(get_ints(at, op_c, "shape", &shp));
    int64_t n = 1;
    for (int64_t d : shp) n *= d;
    RB_REQUIRE(n == x[0]->numel() && shp.size() <= 8, "reshape: cannot reshape " + shape_str(x[0]) + " to " + at["shape"]);
    RB_TRY(buffer_new(c, x[0]->dtype, shp.data(), (int)shp.size(), out));
    if (x[0]->bytes) RB_CUDA(cudaMemcpyAsync((*out)->ptr, x[0]->ptr, x[0]->bytes, cudaMemcpyDeviceToDevice, c->stream));
    return REWB200_OK;
  }
  if (op == "transpose") {
    RB_TRY(need(1));
    std::vector<int64_t> perm;
    RB_TRY(get_ints(at, op_c, "permutation", &perm));
    return op_transpose(c, x[0], perm, out);
  }
  if (op == "broadcastTo") {
    RB_TRY(need(1));
    std::vector<int64_t> shp, bd;
    RB_TRY(get_ints(at, op_c, "output_shape", &shp));
    RB_TRY(get_ints(at, op_c, "broadcast_dimensions", &bd));
    RB_REQUIRE((int)bd.size() == x[0]->ndims && shp.size() <= 8, "broadcastTo: broadcast_dimensions must name every operand axis");
    int64_t istr[8];
    contiguous_strides(x[0]->dims, x[0]->ndims, istr);
    Strided s;
    memset(&s, 0, sizeof(s));
    s.nd = (int)shp.size();
    for (int i = 0; i < s.nd; ++i) s.dims[i] = shp[i];
    for (int i = 0; i < x[0]->ndims; ++i) {
      RB_REQUIRE(bd[i] >= 0 && bd[i] < s.nd, "broadcastTo: dimension out of range");
      RB_REQUIRE(x[0]->dims[i] == shp[bd[i]] || x[0]->dims[i] == 1, "broadcastTo: operand axis " + std::to_string(i) +
                                                                       " does not match output axis " + std::to_string(bd[i]));
      s.in_str[bd[i]] = (x[0]->dims[i] == 1) ? 0 : istr[i];
    }
    contiguous_strides(s.dims, s.nd, s.out_str);
    RB_TRY(buffer_new(c, x[0]->dtype, shp.data(), s.nd, out));
    return run_strided(c, x[0]->ptr, (*out)->ptr, s, dtype_size(x[0]->dtype));
  }
  if (op == "slice") {
    RB_TRY(need(1));
    std::vector<int64_t> st0, lim, str;
    RB_TRY(get_ints(at, op_c, "start_indices", &st0));
    RB_TRY(get_ints(at, op_c, "limit_indices", &lim));
    RB_TRY(get_ints(at, op_c, "strides", &str));
    const int nd = x[0]->ndims;
    RB_REQUIRE((int)st0.size() == nd && (int)lim.size() == nd && (int)str.size() == nd, "slice: index rank mismatch");
    int64_t istr[8], od[8];
    contiguous_strides(x[0]->dims, nd, istr);
    Strided s;
    memset(&s, 0, sizeof(s));
    s.nd = nd;
    for (int i = 0; i < nd; ++i) {
      RB_REQUIRE(str[i] >= 1 && st0[i] >= 0 && lim[i] >= st0[i] && lim[i] <= x[0]->dims[i], "slice: indices out of range");
      od[i] = (lim[i] - st0[i] + str[i] - 1) / str[i];
      s.dims[i] = od[i];
      s.in_str[i] = istr[i] * str[i];
      s.in_off += st0[i] * istr[i];
    }
    contiguous_strides(od, nd, s.out_str);
    RB_TRY(buffer_new(c, x[0]->dtype, od, nd, out));
    return run_strided(c, x[0]->ptr, (*out)->ptr, s, dtype_size(x[0]->dtype));
  }
  if (op == "concat") {
    RB_REQUIRE(n_operands >= 1, "concat: needs at least one operand");
    std::vector<int64_t> dimv;
    RB_TRY(get_ints(at, op_c, "dimension", &dimv));
    RB_REQUIRE(dimv.size() == 1 && dimv[0] >= 0 && dimv[0] < x[0]->ndims, "concat: dimension out of range");
    const int dim = (int)dimv[0], nd = x[0]->ndims;
    int64_t od[8];
    for (int i = 0; i < nd; ++i) od[i] = x[0]->dims[i];
    od[dim] = 0;
    for (int k = 0; k < n_operands; ++k) {
      RB_REQUIRE(x[k]->ndims == nd && x[k]->dtype == x[0]->dtype, "concat: rank or dtype mismatch");
      for (int i = 0; i < nd; ++i) RB_REQUIRE(i == dim || x[k]->dims[i] == x[0]->dims[i], "concat: shape mismatch off the concat axis");
      od[dim] += x[k]->dims[dim];
    }
    RB_TRY(buffer_new(c, x[0]->dtype, od, nd, out));
    int64_t ostr[8], offset = 0;
    contiguous_strides(od, nd, ostr);
    for (int k = 0; k < n_operands; ++k) {
      Strided s;
      memset(&s, 0, sizeof(s));
      s.nd = nd;
      for (int i = 0; i < nd; ++i) {
        s.dims[i] = x[k]->dims[i];
        s.out_str[i] = ostr[i];
      }
      contiguous_strides(x[k]->dims, nd, s.in_str);
      s.out_off = offset * ostr[dim];
      RB_TRY(run_strided(c, x[k]->ptr, (*out)->ptr, s, dtype_size(x[0]->dtype)));
      offset += x[k]->dims[dim];
    }
    return REWB200_OK;
  }
  if (op == "iota") {
    RB_TRY(need(0));
    std::vector<int64_t> shp, dimv;
    RB_TRY(get_ints(at, op_c, "shape", &shp));
    RB_TRY(get_ints(at, op_c, "dimension", &dimv));
    const int dt = dtype_from_name(at.count("dtype") ? at["dtype"] : "int32");
    RB_REQUIRE(dimv.size() == 1 && dimv[0] >= 0 && dimv[0] < (int64_t)shp.size() && shp.size() <= 8, "iota: dimension out of range");
    RB_REQUIRE(dt == REWB200_I32 || dt == REWB200_F32, "iota: dtype must be int32 or float32");
    RB_TRY(buffer_new(c, dt, shp.data(), (int)shp.size(), out));
    int64_t inner = 1, n = 1;
    for (size_t i = 0; i < shp.size(); ++i) {
      n *= shp[i];
      if ((int64_t)i > dimv[0]) inner *= shp[i];
    }
    if (dt == REWB200_I32) LAUNCH1D(iota_kernel<int>, n, (int*)(*out)->ptr, n, inner, shp[dimv[0]]);
    else LAUNCH1D(iota_kernel<float>, n, (float*)(*out)->ptr, n, inner, shp[dimv[0]]);
    return REWB200_OK;
  }
  if (op == "compare") {
    RB_TRY(need(2));
    static const std::map<std::string, int> dirs = {{"LT", C_LT}, {"LE", C_LE}, {"GT", C_GT}, {"GE", C_GE}, {"EQ", C_EQ}, {"NE", C_NE}};
    RB_REQUIRE(at.count("comparison_direction") && dirs.count(at["comparison_direction"]),
               "compare: comparison_direction must be one of LT LE GT GE EQ NE");
    RB_REQUIRE(same_shape(x[0], x[1]) && x[0]->dtype == x[1]->dtype, "compare: operands must agree in shape and dtype");
    RB_TRY(buffer_new(c, REWB200_BOOL, x[0]->dims, x[0]->ndims, out));
    const int64_t n = x[0]->numel();
    const int code = dirs.at(at["comparison_direction"]);
    if (x[0]->dtype == REWB200_F32) LAUNCH1D(compare_kernel<float>, n, (const float*)x[0]->ptr, (const float*)x[1]->ptr, (uint8_t*)(*out)->ptr, n, code);
    else if (x[0]->dtype == REWB200_I32) LAUNCH1D(compare_kernel<int>, n, (const int*)x[0]->ptr, (const int*)x[1]->ptr, (uint8_t*)(*out)->ptr, n, code);
    else return fail("compare: dtype must be float32 or int32");
    return REWB200_OK;
  }
  if (op == "select") {
    RB_TRY(need(3));
    RB_REQUIRE(x[0]->dtype == REWB200_BOOL && same_shape(x[0], x[1]) && same_shape(x[1], x[2]) && x[1]->dtype == x[2]->dtype,
               "select: predicate must be bool and all shapes must agree");
    RB_TRY(buffer_new(c, x[1]->dtype, x[1]->dims, x[1]->ndims, out));
    const int64_t n = x[1]->numel();
    const size_t es = dtype_size(x[1]->dtype);
    if (es == 4) LAUNCH1D(select_kernel<uint32_t>, n, (const uint8_t*)x[0]->ptr, (const uint32_t*)x[1]->ptr, (const uint32_t*)x[2]->ptr, (uint32_t*)(*out)->ptr, n);
    else if (es == 2) LAUNCH1D(select_kernel<uint16_t>, n, (const uint8_t*)x[0]->ptr, (const uint16_t*)x[1]->ptr, (const uint16_t*)x[2]->ptr, (uint16_t*)(*out)->ptr, n);
    else return fail("select: unsupported element size");
    return REWB200_OK;
  }
  if (op == "astype") {
    RB_TRY(need(1));
    const int dt = dtype_from_name(at.count("dtype") ? at["dtype"] : "");
    RB_REQUIRE(dt >= 0, "astype: unknown dtype '" + at["dtype"] + "'");
    RB_TRY(buffer_new(c, dt, x[0]->dims, x[0]->ndims, out));
    const int64_t n = x[0]->numel();
    const int sd = x[0]->dtype;
    void* o = (*out)->ptr;
    if (sd == dt) { if (x[0]->bytes) RB_CUDA(cudaMemcpyAsync(o, x[0]->ptr, x[0]->bytes, cudaMemcpyDeviceToDevice, c->stream)); }
    else if (sd == REWB200_F32 && dt == REWB200_BF16) LAUNCH1D(f32_to_bf16_kernel, n, (const float*)x[0]->ptr, (bf16*)o, n);
    else if (sd == REWB200_BF16 && dt == REWB200_F32) LAUNCH1D(bf16_to_f32_kernel, n, (const bf16*)x[0]->ptr, (float*)o, n);
    else if (sd == REWB200_I32 && dt == REWB200_F32) LAUNCH1D((convert_kernel<int, float>), n, (const int*)x[0]->ptr, (float*)o, n);
    else if (sd == REWB200_F32 && dt == REWB200_I32) LAUNCH1D((convert_kernel<float, int>), n, (const float*)x[0]->ptr, (int*)o, n);
    else if (sd == REWB200_BOOL && dt == REWB200_F32) LAUNCH1D((convert_kernel<uint8_t, float>), n, (const uint8_t*)x[0]->ptr, (float*)o, n);
    else if (sd == REWB200_BOOL && dt == REWB200_I32) LAUNCH1D((convert_kernel<uint8_t, int>), n, (const uint8_t*)x[0]->ptr, (int*)o, n);
    else if (sd == REWB200_I32 && dt == REWB200_I64) LAUNCH1D((convert_kernel<int, long long>), n, (const int*)x[0]->ptr, (long long*)o, n);
    else if (sd == REWB200_I64 && dt == REWB200_I32) LAUNCH1D((convert_kernel<long long, int>), n, (const long long*)x[0]->ptr, (int*)o, n);
    else return fail("astype: conversion not supported by the rew_b200 backend");
    return REWB200_OK;
  }
  if (op == "reduceSum" || op == "reduceMax") {
    RB_TRY(need(1));
    // src/rew/ops/reduce.nim:66-69: reductions are float32 only
    RB_REQUIRE(x[0]->dtype == REWB200_F32, op + ": only float32 is supported (v1)");
    std::vector<int64_t> dims;
    RB_TRY(get_ints(at, op_c, "dims", &dims));
    const int nd = x[0]->ndims;
    std::vector<bool> red(nd, false);
    for (int64_t d : dims) {
      RB_REQUIRE(d >= 0 && d < nd, op + ": dimension out of range");
      red[d] = true;
    }
    std::vector<int64_t> perm, od;
    int64_t len = 1;
    for (int i = 0; i < nd; ++i)
      if (!red[i]) {
        perm.push_back(i);
        od.push_back(x[0]->dims[i]);
      }
    for (int i = 0; i < nd; ++i)
      if (red[i]) {
        perm.push_back(i);
        len *= x[0]->dims[i];
      }
    RB_REQUIRE(len > 0, op + ": empty reduction");
    rewb200_buffer* t = nullptr;
    RB_TRY(op_transpose(c, x[0], perm, &t));
    int st = buffer_new(c, REWB200_F32, od.data(), (int)od.size(), out);
    if (st == REWB200_OK) {
      const int64_t rows = (*out)->numel();
      if (rows > 0) {
        reduce_rows_kernel<<<(unsigned)rows, 128, 0, c->stream>>>((const float*)t->ptr, (float*)(*out)->ptr, len, op == "reduceMax");
        if (cudaGetLastError() != cudaSuccess) st = fail("reduce launch failed");
        ++g_launch_total;
      }
    }
    rewb200_buffer_release(t);
    return st;
  }
  if (op == "dotGeneral") {
    RB_TRY(need(2));
    std::vector<int64_t> lb, rbt, lc, rc;
    RB_TRY(get_ints(at, op_c, "lhs_batching", &lb));
    RB_TRY(get_ints(at, op_c, "rhs_batching", &rbt));
    RB_TRY(get_ints(at, op_c, "lhs_contracting", &lc));
    RB_TRY(get_ints(at, op_c, "rhs_contracting", &rc));
    RB_REQUIRE(x[0]->dtype == REWB200_F32 && x[1]->dtype == REWB200_F32, "dotGeneral: this entry computes float32; use rewb200_linear for bf16");
    RB_REQUIRE(lb.size() == rbt.size() && lc.size() == rc.size(), "dotGeneral: batching/contracting rank mismatch");
    auto arrange = [&](const rewb200_buffer* t, const std::vector<int64_t>& b, const std::vector<int64_t>& k, bool free_first,
                       std::vector<int64_t>* perm, int64_t* nb, int64_t* nf, int64_t* nk, std::vector<int64_t>* free_dims) -> int {
      std::vector<bool> used(t->ndims, false);
      *nb = *nf = *nk = 1;
      for (int64_t d : b) { RB_REQUIRE(d >= 0 && d < t->ndims, "dotGeneral: dimension out of range"); used[d] = true; perm->push_back(d); *nb *= t->dims[d]; }
      std::vector<int64_t> fr;
      for (int64_t d : k) { RB_REQUIRE(d >= 0 && d < t->ndims && !used[d], "dotGeneral: dimension out of range"); used[d] = true; *nk *= t->dims[d]; }
      for (int i = 0; i < t->ndims; ++i) if (!used[i]) { fr.push_back(i); *nf *= t->dims[i]; free_dims->push_back(t->dims[i]); }
      if (free_first) { perm->insert(perm->end(), fr.begin(), fr.end()); perm->insert(perm->end(), k.begin(), k.end()); }
      else { perm->insert(perm->end(), k.begin(), k.end()); perm->insert(perm->end(), fr.begin(), fr.end()); }
      return REWB200_OK;
    };
    std::vector<int64_t> pl, pr, fl, fr;
    int64_t nbl, M, Kl, nbr, N, Kr;
    RB_TRY(arrange(x[0], lb, lc, true, &pl, &nbl, &M, &Kl, &fl));
    RB_TRY(arrange(x[1], rbt, rc, false, &pr, &nbr, &N, &Kr, &fr));
    RB_REQUIRE(nbl == nbr && Kl == Kr, "dotGeneral: batch or contracting sizes differ: " + shape_str(x[0]) + " . " + shape_str(x[1]));
    rewb200_buffer *a = nullptr, *b = nullptr;
    RB_TRY(op_transpose(c, x[0], pl, &a));
    int st = op_transpose(c, x[1], pr, &b);
    std::vector<int64_t> od;
    for (int64_t d : lb) od.push_back(x[0]->dims[d]);
    od.insert(od.end(), fl.begin(), fl.end());
    od.insert(od.end(), fr.begin(), fr.end());
    if (st == REWB200_OK && od.size() > 8) st = fail("dotGeneral: result rank above 8");
    if (st == REWB200_OK) st = buffer_new(c, REWB200_F32, od.data(), (int)od.size(), out);
    for (int64_t bi = 0; st == REWB200_OK && bi < nbl; ++bi)
      st = gemm_f32_launch(c, (const float*)a->ptr + bi * M * Kl, (const float*)b->ptr + bi * Kl * N, nullptr,
                           (float*)(*out)->ptr + bi * M * N, M, Kl, N);
    rewb200_buffer_release(a);
    rewb200_buffer_release(b);
    return st;
  }
  if (op == "topK") {
    RB_TRY(need(1));
    RB_REQUIRE(cap >= 2, "topK: needs room for two results (values, indices)");
    RB_REQUIRE(x[0]->dtype == REWB200_F32 && x[0]->ndims >= 1, "topK: operand must be float32 with rank >= 1");
    std::vector<int64_t> kv;
    RB_TRY(get_ints(at, op_c, "k", &kv));
    const int64_t n = x[0]->dims[x[0]->ndims - 1];
    RB_REQUIRE(kv.size() == 1 && kv[0] > 0, "topK: k must be positive, got " + at["k"]);
    RB_REQUIRE(kv[0] <= n, "topK: k " + std::to_string(kv[0]) + " > dim size " + std::to_string(n));
    if (at.count("dimension")) {
      std::vector<int64_t> dv;
      RB_TRY(get_ints(at, op_c, "dimension", &dv));
      RB_REQUIRE(dv.size() == 1 && (dv[0] == -1 || dv[0] == x[0]->ndims - 1), "topK: only the last dimension is supported");
    }
    int64_t od[8];
    for (int i = 0; i < x[0]->ndims; ++i) od[i] = x[0]->dims[i];
    od[x[0]->ndims - 1] = kv[0];
    RB_TRY(buffer_new(c, REWB200_F32, od, x[0]->ndims, &out[0]));
    RB_TRY(buffer_new(c, REWB200_I32, od, x[0]->ndims, &out[1]));
    *n_out = 2;
    const int64_t rows = n ? x[0]->numel() / n : 0;
    if (rows > 0) {
      topk_rows_kernel<<<(unsigned)rows, 256, 0, c->stream>>>((const float*)x[0]->ptr, n, (int)kv[0], (float*)out[0]->ptr, (int*)out[1]->ptr);
      RB_CUDA(cudaGetLastError());
      ++g_launch_total;
    }
    return REWB200_OK;
  }
  return fail("eager op '" + op + "': not supported by the rew_b200 backend");
}
