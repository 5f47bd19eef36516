// Gated linear attention as a recurrence over a matrix state.
//
// Per request and head the state S [dim, vdim] (float32, one slot per live request) follows
//     S_t = diag(a_t) S_{t-1} + k_t v_t^T,        o_t = S_t^T (q_t * q_scale),
// where the decay a_t [dim] in (0, 1) acts on the rows of S (the key channels):
//     a_t = sigmoid(z_t + b)^(1 / tau) = exp(logsigmoid(z_t + b) / tau).
// The same kernel serves prompts, portions of prompts and single decoded tokens: it reads the
// state its request left, walks the entry's tokens in order and writes the state back, so a
// token's output is the same arithmetic however the tokens were cut into steps or batched.
// Everything that enters the recurrence is float32: decay, its logarithm, state, sums; q, k, v
// are read in the element kind of the projections.
//
// Work split: a CTA owns one (entry, head, tile of VT value columns); thread (j, g) keeps the 8 x 4
// block of the state at rows d = 8 g .. 8 g + 7, columns 4 j .. 4 j + 3 in registers, so that every
// value of q, k, a and v it loads from shared memory serves four or eight multiply-adds.  Tokens are
// staged in shared memory CHUNK at a time (q, k, a once per CTA); each thread updates its block and
// keeps partial outputs per token, and the partial sums of the row groups are added in the order of g
// after every chunk.
//
// Long entries (prompts) are cut into segments of seg_len tokens that run side by side, since one
// entry alone offers only heads x vdim x dim / 16 threads: pass 1 walks every segment from a zero
// state and keeps its end state L and the product A of its decays; a small kernel chains them,
// S_start(s + 1) = diag(A_s) S_start(s) + L_s, from the request's state, which it also brings up to
// date; pass 2 walks every segment again from its true start state and writes the outputs.  This
// regroups the float32 sums of the recurrence (a token's result then depends, within rounding, on
// where its segment begins); entries of up to seg_len tokens, decoded tokens among them, are one
// segment and take the single pass.
#include "common.cuh"

namespace {

constexpr int ROWS = 8;       // state rows per thread
constexpr int COLS = 4;       // state columns per thread
constexpr int CHUNK = 8;      // tokens staged at a time
constexpr int MAX_GROUPS = 32;

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <typename T, int VT>
__global__ void __launch_bounds__(VT / COLS * MAX_GROUPS)
gla_scan_kernel(float* __restrict__ out, long long out_stride, const T* __restrict__ q, const T* __restrict__ k,
                const T* __restrict__ v, long long qkv_stride, const float* __restrict__ z, long long z_stride,
                const float* __restrict__ z_bias, float inv_tau, float q_scale, float* __restrict__ state,
                const int* __restrict__ state_slots, const int* __restrict__ cu_tokens, int heads, int dim, int vdim,
                int seg_len, int max_segs, int mode, float* __restrict__ seg_state, float* __restrict__ seg_decay,
                int z_is_decay) {
  extern __shared__ __align__(16) float smem[];
  pdl_launch_dependents();
  pdl_wait();
  // mode 0: the whole entry from its request's state, which is written back.  mode 1 (pass 1 of a segmented run):
  // a segment from zero, no outputs; its end state and decay product go to seg_state / seg_decay.  mode 2 (pass 2):
  // a segment from seg_state (by then its true start), outputs only.
  constexpr int TX = VT / COLS;               // threads along the columns
  const int groups = blockDim.y, dpad = groups * ROWS;
  float* q_s = smem;                          // [CHUNK][dpad]
  float* k_s = q_s + CHUNK * dpad;
  float* a_s = k_s + CHUNK * dpad;
  float* v_s = a_s + CHUNK * dpad;            // [CHUNK][VT]
  float* part = v_s + CHUNK * VT;             // [CHUNK][groups][VT]
  const int j = threadIdx.x, g = threadIdx.y;
  const int tid = g * TX + j, nthreads = TX * groups;
  const int entry = blockIdx.z / max_segs, seg = blockIdx.z % max_segs, head = blockIdx.y;
  const int col0 = blockIdx.x * VT + j * COLS;
  int t0 = cu_tokens[entry], t1 = cu_tokens[entry + 1];
  size_t seg_index = 0;
  if (mode != 0) {
    if (seg * seg_len >= t1 - t0) return;
    for (int e = 0; e < entry; ++e) seg_index += (cu_tokens[e + 1] - cu_tokens[e] + seg_len - 1) / seg_len;
    seg_index += seg;
    t0 += seg * seg_len;
    t1 = min(t1, t0 + seg_len);
  }
  float* S_g = mode == 0 ? state + (((size_t)state_slots[entry] * heads + head) * dim) * vdim
                         : seg_state + ((seg_index * heads + head) * dim) * vdim;

  float S[ROWS][COLS], A[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int d = g * ROWS + r;
#pragma unroll
    for (int c = 0; c < COLS; ++c)
      S[r][c] = (mode != 1 && d < dim && col0 + c < vdim) ? S_g[(size_t)d * vdim + col0 + c] : 0.f;
    A[r] = 1.f;
  }
  for (int c0 = t0; c0 < t1; c0 += CHUNK) {
    const int n = min(CHUNK, t1 - c0);
    __syncthreads();                          // the previous chunk's partial sums have been read
    for (int c = 0; c < n; ++c) {
      for (int d = tid; d < dpad; d += nthreads) {
        float qv = 0.f, kv = 0.f, av = 0.f;
        if (d < dim) {
          const size_t at = (size_t)(c0 + c) * qkv_stride + (size_t)head * dim + d;
          if (mode != 1) qv = to_f32(q[at]) * q_scale;
          kv = to_f32(k[at]);
          const float zz = z[(size_t)(c0 + c) * z_stride + (size_t)head * dim + d];
          // the two passes of a segmented run read the decay itself, made once by gla_decay_kernel
          av = z_is_decay ? zz : expf(log_sigmoid(zz + (z_bias ? z_bias[head * dim + d] : 0.f)) * inv_tau);
        }
        q_s[c * dpad + d] = qv; k_s[c * dpad + d] = kv; a_s[c * dpad + d] = av;
      }
    }
    for (int idx = tid; idx < n * VT; idx += nthreads) {
      const int c = idx / VT, jj = idx % VT, cc = blockIdx.x * VT + jj;
      v_s[idx] = cc < vdim ? to_f32(v[(size_t)(c0 + c) * qkv_stride + (size_t)head * vdim + cc]) : 0.f;
    }
    __syncthreads();
    for (int c = 0; c < n; ++c) {
      // the thread's 8 rows of k, a (and q) and its 4 values of v: 16-byte loads, shared by the threads of a row group
      const float4 v4 = *reinterpret_cast<const float4*>(v_s + c * VT + j * COLS);
      const float vv[COLS] = {v4.x, v4.y, v4.z, v4.w};
      float kc[ROWS], ac[ROWS], qc[ROWS];
#pragma unroll
      for (int r = 0; r < ROWS; r += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(k_s + c * dpad + g * ROWS + r);
        const float4 a4 = *reinterpret_cast<const float4*>(a_s + c * dpad + g * ROWS + r);
        kc[r] = k4.x; kc[r + 1] = k4.y; kc[r + 2] = k4.z; kc[r + 3] = k4.w;
        ac[r] = a4.x; ac[r + 1] = a4.y; ac[r + 2] = a4.z; ac[r + 3] = a4.w;
        if (mode != 1) {
          const float4 q4 = *reinterpret_cast<const float4*>(q_s + c * dpad + g * ROWS + r);
          qc[r] = q4.x; qc[r + 1] = q4.y; qc[r + 2] = q4.z; qc[r + 3] = q4.w;
        }
      }
      if (mode == 1) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
#pragma unroll
          for (int cc = 0; cc < COLS; ++cc) S[r][cc] = fmaf(ac[r], S[r][cc], kc[r] * vv[cc]);
          A[r] *= ac[r];
        }
        continue;
      }
      float o[COLS] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
#pragma unroll
        for (int cc = 0; cc < COLS; ++cc) {
          S[r][cc] = fmaf(ac[r], S[r][cc], kc[r] * vv[cc]);
          o[cc] = fmaf(S[r][cc], qc[r], o[cc]);
        }
      }
      *reinterpret_cast<float4*>(part + (c * groups + g) * VT + j * COLS) = make_float4(o[0], o[1], o[2], o[3]);
    }
    if (mode == 1) continue;
    __syncthreads();
    for (int idx = tid; idx < n * VT; idx += nthreads) {
      const int c = idx / VT, jj = idx % VT, cc = blockIdx.x * VT + jj;
      if (cc >= vdim) continue;
      float o = 0.f;
      for (int gg = 0; gg < groups; ++gg) o += part[(c * groups + gg) * VT + jj];
      out[(size_t)(c0 + c) * out_stride + (size_t)head * vdim + cc] = o;
    }
  }
  if (mode == 2) return;
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int d = g * ROWS + r;
    if (d >= dim) continue;
#pragma unroll
    for (int c = 0; c < COLS; ++c)
      if (col0 + c < vdim) S_g[(size_t)d * vdim + col0 + c] = S[r][c];
    if (mode == 1 && blockIdx.x == 0 && j == 0) seg_decay[(seg_index * heads + head) * dim + d] = A[r];
  }
}

// ---- the two passes of a segmented run, with the next chunk in flight -------------------------------------
// Same work split and arithmetic as gla_scan_kernel in modes 1 and 2, but a chunk's q, k, decays and v are brought
// into shared memory as they lie in global memory by asynchronous 16-byte copies (cp.async), two stages deep, so that
// the copies of chunk i + 1 run under the multiply-adds of chunk i; the values are widened to float32 when they are
// read from shared memory, and q's scale is applied to the output sums.  Needs rows on the 16-byte grid (dim a
// multiple of 8, vdim a multiple of the tile) and the decays made beforehand (gla_decay_kernel).
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename T> __device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 f = *reinterpret_cast<const float4*>(p);
  v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
  v[0] = __low2float(h[0]); v[1] = __high2float(h[0]); v[2] = __low2float(h[1]); v[3] = __high2float(h[1]);
}

template <typename T, int VT>
__global__ void __launch_bounds__(VT / COLS * MAX_GROUPS)
gla_scan_pipe_kernel(float* __restrict__ out, long long out_stride, const T* __restrict__ q, const T* __restrict__ k,
                     const T* __restrict__ v, long long qkv_stride, const float* __restrict__ a, long long a_stride,
                     float q_scale, const int* __restrict__ cu_tokens, int heads, int dim, int vdim, int seg_len,
                     int max_segs, int mode, float* __restrict__ seg_state, float* __restrict__ seg_decay) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_launch_dependents();
  pdl_wait();
  constexpr int TX = VT / COLS;
  const int groups = blockDim.y;                       // dim == groups * ROWS here
  const size_t qk_bytes = (size_t)CHUNK * dim * sizeof(T), a_bytes = (size_t)CHUNK * dim * sizeof(float);
  const size_t v_bytes = (size_t)CHUNK * VT * sizeof(T), stage_bytes = 2 * qk_bytes + a_bytes + v_bytes;
  float* part = reinterpret_cast<float*>(smem_raw + 2 * stage_bytes);      // [CHUNK][groups][VT]
  const int j = threadIdx.x, g = threadIdx.y;
  const int tid = g * TX + j, nthreads = TX * groups;
  const int entry = blockIdx.z / max_segs, seg = blockIdx.z % max_segs, head = blockIdx.y;
  const int col0 = blockIdx.x * VT + j * COLS;
  int t0 = cu_tokens[entry], t1 = cu_tokens[entry + 1];
  if (seg * seg_len >= t1 - t0) return;
  size_t seg_index = seg;
  for (int e = 0; e < entry; ++e) seg_index += (cu_tokens[e + 1] - cu_tokens[e] + seg_len - 1) / seg_len;
  t0 += seg * seg_len;
  t1 = min(t1, t0 + seg_len);
  float* S_g = seg_state + ((seg_index * heads + head) * dim) * vdim;

  auto issue = [&](int c0, int stage) {
    const int n = min(CHUNK, t1 - c0);
    unsigned char* base = smem_raw + stage * stage_bytes;
    const int rv = dim * (int)sizeof(T) / 16, av = dim * 4 / 16, vv = VT * (int)sizeof(T) / 16;
    for (int idx = tid; idx < n * rv; idx += nthreads) {
      const int c = idx / rv, x = idx % rv;
      const size_t src = (size_t)(c0 + c) * qkv_stride + (size_t)head * dim;
      if (mode != 1) cp_async16(base + (size_t)c * dim * sizeof(T) + x * 16, reinterpret_cast<const char*>(q + src) + x * 16);
      cp_async16(base + qk_bytes + (size_t)c * dim * sizeof(T) + x * 16, reinterpret_cast<const char*>(k + src) + x * 16);
    }
    for (int idx = tid; idx < n * av; idx += nthreads) {
      const int c = idx / av, x = idx % av;
      cp_async16(base + 2 * qk_bytes + (size_t)c * dim * 4 + x * 16,
                 reinterpret_cast<const char*>(a + (size_t)(c0 + c) * a_stride + (size_t)head * dim) + x * 16);
    }
    for (int idx = tid; idx < n * vv; idx += nthreads) {
      const int c = idx / vv, x = idx % vv;
      cp_async16(base + 2 * qk_bytes + a_bytes + (size_t)c * VT * sizeof(T) + x * 16,
                 reinterpret_cast<const char*>(v + (size_t)(c0 + c) * qkv_stride + (size_t)head * vdim + blockIdx.x * VT) + x * 16);
    }
  };

  float S[ROWS][COLS], A[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
#pragma unroll
    for (int c = 0; c < COLS; ++c) S[r][c] = mode == 2 ? S_g[(size_t)(g * ROWS + r) * vdim + col0 + c] : 0.f;
    A[r] = 1.f;
  }
  issue(t0, 0);
  cp_async_commit();
  int stage = 0;
  for (int c0 = t0; c0 < t1; c0 += CHUNK, stage ^= 1) {
    const int n = min(CHUNK, t1 - c0);
    if (c0 + CHUNK < t1) issue(c0 + CHUNK, stage ^ 1);     // the other stage was read two iterations ago (barrier below)
    cp_async_commit();
    cp_async_wait<1>();                                    // this chunk's copies have landed (the newest group may fly)
    __syncthreads();
    const unsigned char* base = smem_raw + stage * stage_bytes;
    const T* q_s = reinterpret_cast<const T*>(base);
    const T* k_s = reinterpret_cast<const T*>(base + qk_bytes);
    const float* a_s = reinterpret_cast<const float*>(base + 2 * qk_bytes);
    const T* v_s = reinterpret_cast<const T*>(base + 2 * qk_bytes + a_bytes);
    for (int c = 0; c < n; ++c) {
      float vv[COLS], kc[ROWS], ac[ROWS], qc[ROWS];
      load4<T>(v_s + c * VT + j * COLS, vv);
      Vec8<T>::load(k_s + c * dim + g * ROWS, kc);
      Vec8<float>::load(a_s + c * dim + g * ROWS, ac);
      if (mode == 1) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
#pragma unroll
          for (int cc = 0; cc < COLS; ++cc) S[r][cc] = fmaf(ac[r], S[r][cc], kc[r] * vv[cc]);
          A[r] *= ac[r];
        }
        continue;
      }
      Vec8<T>::load(q_s + c * dim + g * ROWS, qc);
      float o[COLS] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
#pragma unroll
        for (int cc = 0; cc < COLS; ++cc) {
          S[r][cc] = fmaf(ac[r], S[r][cc], kc[r] * vv[cc]);
          o[cc] = fmaf(S[r][cc], qc[r], o[cc]);
        }
      }
      *reinterpret_cast<float4*>(part + (c * groups + g) * VT + j * COLS) = make_float4(o[0], o[1], o[2], o[3]);
    }
    __syncthreads();                                       // the stage is free for the copies after next; part is complete
    if (mode == 1) continue;
    for (int idx = tid; idx < n * VT; idx += nthreads) {
      const int c = idx / VT, jj = idx % VT;
      float o = 0.f;
      for (int gg = 0; gg < groups; ++gg) o += part[(c * groups + gg) * VT + jj];
      out[(size_t)(c0 + c) * out_stride + (size_t)head * vdim + blockIdx.x * VT + jj] = o * q_scale;
    }
    // part is read here and written again only after the next iteration's first barrier
  }
  cp_async_wait<0>();
  if (mode == 2) return;
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int d = g * ROWS + r;
#pragma unroll
    for (int c = 0; c < COLS; ++c) S_g[(size_t)d * vdim + col0 + c] = S[r][c];
    if (blockIdx.x == 0 && j == 0) seg_decay[(seg_index * heads + head) * dim + d] = A[r];
  }
}

// z <- sigmoid(z + bias)^(1 / tau) in place: the decays of a step, made once where several CTAs and two passes read them.
__global__ void gla_decay_kernel(float* __restrict__ z, long long z_stride, const float* __restrict__ z_bias, float inv_tau,
                                 int cols, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / cols;
    const int c = (int)(i - t * cols);
    float* at = z + t * z_stride + c;
    *at = expf(log_sigmoid(*at + (z_bias ? z_bias[c] : 0.f)) * inv_tau);
  }
}

// Chains the segments of every entry: seg_state[s] holds the segment's end state from zero on entry and its true start
// state on exit; the request's state moves to the end of the entry.  One thread per element of the state.
__global__ void gla_chain_kernel(float* __restrict__ seg_state, const float* __restrict__ seg_decay, float* __restrict__ state,
                                 const int* __restrict__ state_slots, const int* __restrict__ cu_tokens, int heads, int dim,
                                 int vdim, int seg_len) {
  pdl_launch_dependents();
  pdl_wait();
  const int entry = blockIdx.y;
  const size_t per = (size_t)heads * dim * vdim;
  const size_t el = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (el >= per) return;
  size_t seg0 = 0;
  for (int e = 0; e < entry; ++e) seg0 += (cu_tokens[e + 1] - cu_tokens[e] + seg_len - 1) / seg_len;
  const int n_seg = (cu_tokens[entry + 1] - cu_tokens[entry] + seg_len - 1) / seg_len;
  const size_t row = el / vdim;                       // (head, d)
  float* S_g = state + (size_t)state_slots[entry] * per + el;
  float S = *S_g;
  for (int s = 0; s < n_seg; ++s) {
    float* at = seg_state + (seg0 + s) * per + el;
    const float local = *at;
    *at = S;
    S = fmaf(seg_decay[(seg0 + s) * heads * dim + row], S, local);
  }
  *S_g = S;
}

}  // namespace

// out float32 [tokens, out_stride] with head h at column h * vdim.  q, k (head h at column h * dim) and v (head h at
// column h * vdim) are rows of the element kind, qkv_stride elements apart.  z float32 [tokens, z_stride], the
// decay's pre-activation, head h at column h * dim; z_bias float32 [heads * dim] or null.  state float32
// [slots, heads, dim, vdim]; state_slots [entries]; cu_tokens [entries + 1]: entry e owns tokens cu[e] .. cu[e+1]-1.
// A launch that 32 columns a tile would leave with fewer CTAs than SMs takes narrower tiles (16, 8); the sums of
// a column do not depend on the tile's width.
// seg_len > 0: entries run as segments of seg_len tokens in two passes (see the head of the file); n_tokens is then the
// step's number of tokens, seg_state float32 [n_tokens / seg_len + n_entries, heads, dim, vdim] and seg_decay
// [same, heads, dim] scratch, and z is overwritten with the decays.  seg_len 0: one pass.
LLMK_API int llmk_gla_scan(float* out, long long out_stride, const void* q, const void* k, const void* v,
                           long long qkv_stride, float* z, long long z_stride, const float* z_bias, float tau,
                           float q_scale, float* state, const int* state_slots, const int* cu_tokens, int n_entries,
                           int heads, int dim, int vdim, int dtype, cudaStream_t stream, int n_tokens, int seg_len,
                           float* seg_state, float* seg_decay) {
  if (n_entries == 0) return 0;
  LLMK_REQUIRE(seg_len >= 0 && (seg_len == 0 || (seg_state && seg_decay && n_tokens > 0)), "gla_scan: segments need their scratch");
  // the longest entry has at most n_tokens - (n_entries - 1) tokens: a bound that depends on the step's sizes alone
  const int max_segs = seg_len ? (n_tokens - (n_entries - 1) + seg_len - 1) / seg_len : 1;
  LLMK_REQUIRE((long long)n_entries * max_segs <= 65535, "gla_scan: too many segments for one launch");
  LLMK_REQUIRE(heads > 0 && dim > 0 && vdim > 0, "gla_scan: sizes must be positive");
  LLMK_REQUIRE(dim <= ROWS * MAX_GROUPS, "gla_scan: key size %d exceeds %d", dim, ROWS * MAX_GROUPS);
  LLMK_REQUIRE(tau > 0.f, "gla_scan: tau must be positive");
  LLMK_REQUIRE(n_entries <= 65535 && heads <= 65535, "gla_scan: too many entries or heads for one launch");
  const int groups = (dim + ROWS - 1) / ROWS;
  const long long wide = (long long)((vdim + 31) / 32) * heads * n_entries * (seg_len ? (n_tokens + seg_len - 1) / seg_len : 1);
  const int sms = llmk_sm_count();
  const int vt = wide >= sms ? 32 : (wide * 2 >= sms ? 16 : 8);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    auto launch = [&](auto kern, int VT, int mode) {
      const size_t smem = sizeof(float) * ((size_t)CHUNK * groups * ROWS * 3 + (size_t)CHUNK * VT + (size_t)CHUNK * groups * VT);
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      return launch_kernel(kern, dim3((vdim + VT - 1) / VT, heads, n_entries * max_segs), dim3(VT / COLS, groups), smem, stream, out,
                           out_stride, (const T*)q, (const T*)k, (const T*)v, qkv_stride, z, z_stride, z_bias, 1.f / tau, q_scale,
                           state, state_slots, cu_tokens, heads, dim, vdim, seg_len, max_segs, mode, seg_state, seg_decay,
                           seg_len ? 1 : 0);
    };
    // the passes of a segmented run take the kernel with asynchronous copies where every row lies on the 16-byte grid
    const bool pipe = seg_len > 0 && dim % 8 == 0 && vdim % vt == 0 && qkv_stride % 8 == 0 && z_stride % 4 == 0 &&
                      (uintptr_t)q % 16 == 0 && (uintptr_t)k % 16 == 0 && (uintptr_t)v % 16 == 0 && (uintptr_t)z % 16 == 0;
    auto launch_pipe = [&](auto kern, int VT, int mode) {
      const size_t stage = 2 * (size_t)CHUNK * dim * sizeof(T) + (size_t)CHUNK * dim * sizeof(float) + (size_t)CHUNK * VT * sizeof(T);
      const size_t smem = 2 * stage + sizeof(float) * (size_t)CHUNK * groups * VT;
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      return launch_kernel(kern, dim3(vdim / VT, heads, n_entries * max_segs), dim3(VT / COLS, groups), smem, stream, out, out_stride,
                           (const T*)q, (const T*)k, (const T*)v, qkv_stride, (const float*)z, z_stride, q_scale, cu_tokens, heads, dim,
                           vdim, seg_len, max_segs, mode, seg_state, seg_decay);
    };
    auto pass = [&](int mode) {
      if (pipe) {
        if (vt == 32) launch_pipe(gla_scan_pipe_kernel<T, 32>, 32, mode);
        else if (vt == 16) launch_pipe(gla_scan_pipe_kernel<T, 16>, 16, mode);
        else launch_pipe(gla_scan_pipe_kernel<T, 8>, 8, mode);
        return;
      }
      if (vt == 32) launch(gla_scan_kernel<T, 32>, 32, mode);
      else if (vt == 16) launch(gla_scan_kernel<T, 16>, 16, mode);
      else launch(gla_scan_kernel<T, 8>, 8, mode);
    };
    if (seg_len == 0) {
      pass(0);
    } else {
      const size_t total = (size_t)n_tokens * heads * dim;
      size_t blocks = (total + 255) / 256;
      if (blocks > (size_t)sms * 8) blocks = (size_t)sms * 8;
      launch_kernel(gla_decay_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, z, z_stride, z_bias, 1.f / tau, heads * dim, total);
      pass(1);
      const size_t per = (size_t)heads * dim * vdim;
      launch_kernel(gla_chain_kernel, dim3((unsigned)((per + 255) / 256), n_entries), dim3(256), 0, stream, seg_state,
                    (const float*)seg_decay, state, state_slots, cu_tokens, heads, dim, vdim, seg_len);
      pass(2);
    }
    LLMK_LAUNCH_CHECK("gla_scan");
  });
}
