// Time mixing in the manner of RWKV: a linear recurrence per head whose decay is computed from the data, read
// through mixes of every token with the token before it.
//
// token_shift_mix      out[t, s*sec + c] = x[t, c] + (prev[t, c] - x[t, c]) * mu[s, c] for each of n_mix mixes s, where
//                      prev is the row before t of the same request: a row of this step, or, for the request's
//                      first row of the step, the last row of the step before, kept in the state (zeros at position 0).
// shift_state_update   moves the last row of every request's run into the state (launched after the mix).
// wkv_scan             per (request, head), state S of K rows (key channels) and V columns, float32:
//                        o_t[v] = sum_k r_t[k] (S[k, v] + u[k] k_t[k] v_t[v])      (the bonus u for the current token only)
//                        S[k, v] <- w_t[k] S[k, v] + k_t[k] v_t[v],   w_t[k] = exp(-exp(d_t[k]))
//                      d_t arrives in float32 (the decay's projection with its bias); exponentials, state and sums
//                      are float32; r, k, v arrive in the activation dtype.
//
// A request's rows of a step are req_first_token[r] .. (as many as carry its index in token_req); its state lives
// in row slots[r] of a float32 pool ([slots, H, V, K]: a head's state column by column), read at the start of the
// run and written back at its end.  A thread holds 16 consecutive rows of one column in registers; the NS threads of
// a column are neighbouring lanes and add their partial sums by shuffles; 16 tokens at a time are staged in shared
// memory.  The order of additions for a token depends on the layer's sizes only.
#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

// Rows t0 .. t1-1 that belong to request r (they come first in the range).  Every thread of the block calls it.
__device__ __forceinline__ int run_length(const int* __restrict__ token_req, int t0, int t1, int r) {
  int n = 0;
  for (int base = t0; base < t1; base += blockDim.x) {
    const int t = base + threadIdx.x;
    n += __syncthreads_count(t < t1 && token_req[t] == r);
  }
  return n;
}

template <typename T>
__global__ void token_shift_mix_kernel(const T* x, int ldx, const float* __restrict__ mu, int n_mix, int D,
                                       const float* state, const int* __restrict__ slots,
                                       const int* __restrict__ positions, const int* __restrict__ token_req,
                                       const int* __restrict__ req_first_token, T* __restrict__ out, int ldo, int sec) {
  const int t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = token_req[t];
  if (r < 0 || c >= D) return;
  pdl_wait();
  pdl_trigger();
  x = after_wait(x);
  state = after_wait(state);
  const float cur = to_f(x[(size_t)t * ldx + c]);
  float prev;
  if (t > req_first_token[r]) prev = to_f(x[(size_t)(t - 1) * ldx + c]);
  else prev = positions[t] > 0 ? state[(size_t)slots[r] * D + c] : 0.f;
  const float diff = prev - cur;
  for (int s = 0; s < n_mix; ++s)
    out[(size_t)t * ldo + (size_t)s * sec + c] = from_f<T>(fmaf(diff, mu[(size_t)s * D + c], cur));
}

template <typename T>
__global__ void shift_state_update_kernel(const T* x, int ldx, int D, float* state, const int* __restrict__ slots,
                                          const int* __restrict__ token_req, const int* __restrict__ req_first_token) {
  pdl_wait();
  pdl_trigger();
  x = after_wait(x);
  const int r = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  const int t0 = req_first_token[r], t1 = req_first_token[r + 1];
  const int n = run_length(token_req, t0, t1, r);
  if (n == 0 || c >= D) return;
  state[(size_t)slots[r] * D + c] = to_f(x[(size_t)(t0 + n - 1) * ldx + c]);
}

// x: [n_tokens, >= D] (activation dtype); mu: float32 [n_mix, D]; state: float32 [slots, D]; out: [n_tokens, n_mix*sec],
// mix s in columns s*sec .. s*sec + D - 1 (sec >= D).
MLXB_EXPORT int mlxb_token_shift_mix(int dtype, const void* x, int ldx, const float* mu, int n_mix, int D, float* state,
                                     const int* slots, const int* positions, const int* token_req,
                                     const int* req_first_token, void* out, int ldo, int sec, int n_tokens, int n_requests,
                                     cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (D <= 0 || n_mix <= 0 || ldx < D || sec < D || ldo < n_mix * sec || n_tokens > 65535 * 32 || n_requests > 65535)
    return mlxb_fail(MLXB_BAD_ARG, "token_shift_mix: %d mixes of width %d, strides %d / %d", n_mix, D, ldx, ldo);
  const int threads = D >= 256 ? 256 : 128;
  const dim3 grid((D + threads - 1) / threads, n_tokens), sgrid((D + threads - 1) / threads, n_requests);
  if (dtype == MLXB_F32) {
    launch_pdl(token_shift_mix_kernel<float>, grid, dim3(threads), 0, stream, (const float*)x, ldx, mu, n_mix, D,
               (const float*)state, slots, positions, token_req, req_first_token, (float*)out, ldo, sec);
    if (int e = mlxb_check_launch("token_shift_mix")) return e;
    launch_pdl(shift_state_update_kernel<float>, sgrid, dim3(threads), 0, stream, (const float*)x, ldx, D, state, slots,
               token_req, req_first_token);
  } else if (dtype == MLXB_BF16) {
    launch_pdl(token_shift_mix_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (const __nv_bfloat16*)x, ldx, mu,
               n_mix, D, (const float*)state, slots, positions, token_req, req_first_token, (__nv_bfloat16*)out, ldo, sec);
    if (int e = mlxb_check_launch("token_shift_mix")) return e;
    launch_pdl(shift_state_update_kernel<__nv_bfloat16>, sgrid, dim3(threads), 0, stream, (const __nv_bfloat16*)x, ldx, D,
               state, slots, token_req, req_first_token);
  } else {
    return mlxb_fail(MLXB_BAD_DTYPE, "token_shift_mix: dtype code %d", dtype);
  }
  return mlxb_check_launch("shift_state_update");
}

// ---------------------------------------------------------------- the recurrence

constexpr int WK_NPT = 16;     // rows of a state column a thread holds
constexpr int WK_SEG = 20;     // floats between the staged runs of 16 rows (keeps 16-byte loads of neighbouring lanes apart)
constexpr int WK_CHUNK = 16;   // tokens staged at a time

template <typename T, int NS, bool VEC>
__global__ void __launch_bounds__(256)
wkv_scan_kernel(const T* rkv, int ld, int r_off, int k_off, int v_off, const float* d_raw, int ldd,
                const float* __restrict__ u, float* state, const int* __restrict__ slots,
                const int* __restrict__ token_req, const int* __restrict__ req_first_token, float* __restrict__ o,
                int ldo, int H, int K, int V, int VB, bool pre) {
  extern __shared__ __align__(16) float wk_sm[];
  constexpr int NP = NS * WK_SEG;
  float* sr = wk_sm;                       // [CHUNK][NP]
  float* sk = sr + WK_CHUNK * NP;          // [CHUNK][NP]
  float* sw = sk + WK_CHUNK * NP;          // [CHUNK][NP]
  float* sv = sw + WK_CHUNK * NP;          // [CHUNK][VB]
  float* sb = sv + WK_CHUNK * VB;          // [CHUNK] sum_k r u k of the token
  const int h = blockIdx.x, r = blockIdx.y, vb = blockIdx.z;
  const int tid = threadIdx.x, nthreads = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
  const int s = tid % NS, vl = tid / NS, v = vb * VB + vl;
  const bool valid = v < V;
  pdl_wait();
  pdl_trigger();
  rkv = after_wait(rkv);
  d_raw = after_wait(d_raw);
  state = after_wait(state);
  const int t0 = req_first_token[r], t1 = req_first_token[r + 1];
  const int n = run_length(token_req, t0, t1, r);
  if (n == 0) return;
  float* st = state + (((size_t)slots[r] * H + h) * V + (valid ? v : 0)) * K;   // this thread's column
  float S[WK_NPT];
#pragma unroll
  for (int i = 0; i < WK_NPT; ++i) {
    const int kk = s * WK_NPT + i;
    S[i] = (valid && kk < K) ? st[kk] : 0.f;
  }
  for (int e = tid; e < 3 * WK_CHUNK * NP; e += nthreads) sr[e] = 0.f;     // rows beyond K stay zero
  const float* uh = u + (size_t)h * K;
  // the staged tokens of a chunk through the recurrence
  auto run_tokens = [&](int c0, int nc) {
#pragma unroll 4
    for (int tok = 0; tok < nc; ++tok) {
      const float* pr = sr + tok * NP + s * WK_SEG;
      const float* pk = sk + tok * NP + s * WK_SEG;
      const float* pw = sw + tok * NP + s * WK_SEG;
      const float vv = sv[tok * VB + vl];
      float a = 0.f;
#pragma unroll
      for (int i = 0; i < WK_NPT; i += 4) {
        const float4 r4 = *reinterpret_cast<const float4*>(pr + i);
        const float4 k4 = *reinterpret_cast<const float4*>(pk + i);
        const float4 w4 = *reinterpret_cast<const float4*>(pw + i);
        a = fmaf(r4.x, S[i], a);
        a = fmaf(r4.y, S[i + 1], a);
        a = fmaf(r4.z, S[i + 2], a);
        a = fmaf(r4.w, S[i + 3], a);
        S[i] = fmaf(w4.x, S[i], k4.x * vv);
        S[i + 1] = fmaf(w4.y, S[i + 1], k4.y * vv);
        S[i + 2] = fmaf(w4.z, S[i + 2], k4.z * vv);
        S[i + 3] = fmaf(w4.w, S[i + 3], k4.w * vv);
      }
#pragma unroll
      for (int off = NS / 2; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
      if (s == 0 && valid) o[(size_t)(t0 + c0 + tok) * ldo + h * V + v] = fmaf(sb[tok], vv, a);
    }
  };
  if (VEC && pre) {
    // One staging item a thread (eight key channels of one token of the chunk) and the chunk after this one asked
    // for before this one goes through the recurrence: the loads are in flight while the tokens are walked.
    const int per_tok = K / 8;
    const bool stager = tid < WK_CHUNK * per_tok;
    const int tok_s = tid / per_tok, kk_s = (tid % per_tok) * 8;
    float uv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) uv[i] = stager ? uh[kk_s + i] : 0.f;
    uint4 nr[2], nk[2];
    float4 nd[2];
    float nv[WK_CHUNK];
    auto fetch = [&](int c0) {
      const int nc = min(WK_CHUNK, n - c0);
      if (stager && tok_s < nc) {
        const size_t row = (size_t)(t0 + c0 + tok_s);
        const T* rp = rkv + row * ld + r_off + h * K + kk_s;
        const T* kp = rkv + row * ld + k_off + h * K + kk_s;
        const float* dp = d_raw + row * ldd + h * K + kk_s;
        nr[0] = *reinterpret_cast<const uint4*>(rp);
        nk[0] = *reinterpret_cast<const uint4*>(kp);
        if (sizeof(T) == 4) {
          nr[1] = *reinterpret_cast<const uint4*>(rp + 4);
          nk[1] = *reinterpret_cast<const uint4*>(kp + 4);
        }
        nd[0] = *reinterpret_cast<const float4*>(dp);
        nd[1] = *reinterpret_cast<const float4*>(dp + 4);
      }
#pragma unroll
      for (int i = 0; i < WK_CHUNK; ++i) {
        const int e = tid + i * nthreads;
        if (e < nc * VB) {
          const int tok = e / VB, c = e - tok * VB;
          nv[i] = vb * VB + c < V ? to_f(rkv[(size_t)(t0 + c0 + tok) * ld + v_off + h * V + vb * VB + c]) : 0.f;
        }
      }
    };
    fetch(0);
    for (int c0 = 0; c0 < n; c0 += WK_CHUNK) {
      const int nc = min(WK_CHUNK, n - c0);
      __syncthreads();
      if (stager) {
        float b = 0.f;
        if (tok_s < nc) {
          float rv[8], kv[8], dv[8];
          if (sizeof(T) == 2) {
            unpack8(nr[0], rv);
            unpack8(nk[0], kv);
          } else {
            *reinterpret_cast<uint4*>(rv) = nr[0];
            *reinterpret_cast<uint4*>(rv + 4) = nr[1];
            *reinterpret_cast<uint4*>(kv) = nk[0];
            *reinterpret_cast<uint4*>(kv + 4) = nk[1];
          }
          *reinterpret_cast<float4*>(dv) = nd[0];
          *reinterpret_cast<float4*>(dv + 4) = nd[1];
          const int at = tok_s * NP + (kk_s / WK_NPT) * WK_SEG + (kk_s % WK_NPT);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            sr[at + i] = rv[i];
            sk[at + i] = kv[i];
            sw[at + i] = expf(-expf(dv[i]));
            b = fmaf(rv[i] * uv[i], kv[i], b);
          }
        }
        // (the stagers are whole warps, and a token's per_tok threads an aligned group of lanes)
        for (int off = per_tok >> 1; off > 0; off >>= 1) b += __shfl_xor_sync(0xffffffffu, b, off);
        if (tok_s < nc && kk_s == 0) sb[tok_s] = b;
      }
#pragma unroll
      for (int i = 0; i < WK_CHUNK; ++i) {
        const int e = tid + i * nthreads;
        if (e < nc * VB) sv[e] = nv[i];
      }
      __syncthreads();
      if (c0 + WK_CHUNK < n) fetch(c0 + WK_CHUNK);
      run_tokens(c0, nc);
    }
  } else
  for (int c0 = 0; c0 < n; c0 += WK_CHUNK) {
    const int nc = min(WK_CHUNK, n - c0);
    __syncthreads();
    if (VEC) {
      // eight key channels of a token a thread: the loads of r, k and the decay's input go out together; the eight
      // threads of a token (neighbouring lanes) add up its bonus term sum_k r u k
      const int per_tok = K / 8;
      for (int e = tid; e < WK_CHUNK * per_tok; e += nthreads) {
        const int tok = e / per_tok, kk = (e - tok * per_tok) * 8;
        float b = 0.f;
        if (tok < nc) {
          const size_t row = (size_t)(t0 + c0 + tok);
          float rv[8], kv[8], dv[8], uv[8];
          const T* rp = rkv + row * ld + r_off + h * K + kk;
          const T* kp = rkv + row * ld + k_off + h * K + kk;
          const float* dp = d_raw + row * ldd + h * K + kk;
          if (sizeof(T) == 2) {
            const uint4 r8 = *reinterpret_cast<const uint4*>(rp), k8 = *reinterpret_cast<const uint4*>(kp);
            unpack8(r8, rv);
            unpack8(k8, kv);
          } else {
            *reinterpret_cast<float4*>(rv) = *reinterpret_cast<const float4*>(rp);
            *reinterpret_cast<float4*>(rv + 4) = *reinterpret_cast<const float4*>(rp + 4);
            *reinterpret_cast<float4*>(kv) = *reinterpret_cast<const float4*>(kp);
            *reinterpret_cast<float4*>(kv + 4) = *reinterpret_cast<const float4*>(kp + 4);
          }
          *reinterpret_cast<float4*>(dv) = *reinterpret_cast<const float4*>(dp);
          *reinterpret_cast<float4*>(dv + 4) = *reinterpret_cast<const float4*>(dp + 4);
          *reinterpret_cast<float4*>(uv) = *reinterpret_cast<const float4*>(uh + kk);
          *reinterpret_cast<float4*>(uv + 4) = *reinterpret_cast<const float4*>(uh + kk + 4);
          const int at = tok * NP + (kk / WK_NPT) * WK_SEG + (kk % WK_NPT);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            sr[at + i] = rv[i];
            sk[at + i] = kv[i];
            sw[at + i] = expf(-expf(dv[i]));
            b = fmaf(rv[i] * uv[i], kv[i], b);
          }
        }
        // (per_tok is a power of two up to 32 here, so a token's threads are an aligned group of lanes)
        for (int off = per_tok >> 1; off > 0; off >>= 1) b += __shfl_xor_sync(0xffffffffu, b, off);
        if (tok < nc && (e % per_tok) == 0) sb[tok] = b;
      }
      for (int e = tid; e < nc * VB; e += nthreads) {
        const int tok = e / VB, c = e - tok * VB;
        sv[e] = vb * VB + c < V ? to_f(rkv[(size_t)(t0 + c0 + tok) * ld + v_off + h * V + vb * VB + c]) : 0.f;
      }
      __syncthreads();
    } else {
      for (int e = tid; e < nc * K; e += nthreads) {
        const int tok = e / K, kk = e - tok * K;
        const size_t row = (size_t)(t0 + c0 + tok);
        const int at = tok * NP + (kk / WK_NPT) * WK_SEG + (kk % WK_NPT);
        sr[at] = to_f(rkv[row * ld + r_off + h * K + kk]);
        sk[at] = to_f(rkv[row * ld + k_off + h * K + kk]);
        sw[at] = expf(-expf(d_raw[row * ldd + h * K + kk]));
      }
      for (int e = tid; e < nc * VB; e += nthreads) {
        const int tok = e / VB, c = e - tok * VB;
        sv[e] = vb * VB + c < V ? to_f(rkv[(size_t)(t0 + c0 + tok) * ld + v_off + h * V + vb * VB + c]) : 0.f;
      }
      __syncthreads();
      for (int tok = warp; tok < nc; tok += nwarps) {
        float b = 0.f;
        for (int kk = lane; kk < K; kk += 32) {
          const int at = tok * NP + (kk / WK_NPT) * WK_SEG + (kk % WK_NPT);
          b = fmaf(sr[at] * uh[kk], sk[at], b);
        }
        b = warp_sum(b);
        if (lane == 0) sb[tok] = b;
      }
      __syncthreads();
    }
    run_tokens(c0, nc);
  }
  if (valid) {
#pragma unroll
    for (int i = 0; i < WK_NPT; ++i) {
      const int kk = s * WK_NPT + i;
      if (kk < K) st[kk] = S[i];
    }
  }
}

// rkv: [n_tokens, .] (activation dtype) holding r and k (H*K columns each from r_off / k_off) and v (H*V columns from
// v_off); d_raw: float32 [n_tokens, >= H*K] at row stride ldd; u: float32 [H, K]; state: float32 [slots, H, V, K];
// o: float32 [n_tokens, H*V] at row stride ldo.
MLXB_EXPORT int mlxb_wkv_scan(int dtype, const void* rkv, int ld, int r_off, int k_off, int v_off, const float* d_raw,
                              int ldd, const float* u, float* state, const int* slots, const int* token_req,
                              const int* req_first_token, float* o, int ldo, int H, int K, int V, int n_requests,
                              cudaStream_t stream) {
  if (n_requests <= 0) return 0;
  if (H <= 0 || K <= 0 || V <= 0 || K > 32 * WK_NPT || n_requests > 65535)
    return mlxb_fail(MLXB_BAD_ARG, "wkv_scan: %d heads with states of %d x %d (at most %d rows)", H, K, V, 32 * WK_NPT);
  int NS = 1;
  while (NS * WK_NPT < K) NS *= 2;
  // few (request, head) pairs: the columns of a pair over several blocks, never below two warps a block
  const long long pairs = (long long)H * n_requests;
  const int sms = mlxb_sm_count();
  int threads = 2 * pairs >= sms ? 256 : (4 * pairs >= sms ? 128 : 64);
  // 16-byte staging: K a power of two from 16 to 256 (a token's K/8 staging threads are an aligned group of lanes)
  const bool vec = K >= 16 && K <= 256 && (K & (K - 1)) == 0 && ld % 8 == 0 && r_off % 8 == 0 && k_off % 8 == 0 && ldd % 4 == 0 &&
                   (((uintptr_t)rkv | (uintptr_t)d_raw | (uintptr_t)u) & 15) == 0;
  if (threads < 2 * NS) threads = 2 * NS;
  const int unit = NS >= 32 ? 1 : 32 / NS;                 // columns that make a whole warp
  int VB = threads / NS;
  const int v_up = (V + unit - 1) / unit * unit;
  if (VB > v_up) VB = v_up;
  threads = VB * NS;
  const dim3 grid(H, n_requests, (V + VB - 1) / VB);
  const bool pre = vec && 2 * K <= threads;      // a staging item a thread: the next chunk is fetched ahead
  const size_t smem = sizeof(float) * ((size_t)WK_CHUNK * (3 * NS * WK_SEG + VB + 1));
#define WK_GO(T, N)                                                                                                  \
  if (smem > 48 * 1024) {                                                                                            \
    cudaError_t e = cudaFuncSetAttribute(wkv_scan_kernel<T, N, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e == cudaSuccess) e = cudaFuncSetAttribute(wkv_scan_kernel<T, N, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e != cudaSuccess) return mlxb_fail((int)e, "wkv_scan: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); \
  }                                                                                                                  \
  if (vec)                                                                                                           \
    launch_pdl(wkv_scan_kernel<T, N, true>, grid, dim3(threads), smem, stream, (const T*)rkv, ld, r_off, k_off, v_off, d_raw, \
               ldd, u, state, slots, token_req, req_first_token, o, ldo, H, K, V, VB, pre);                          \
  else                                                                                                               \
    launch_pdl(wkv_scan_kernel<T, N, false>, grid, dim3(threads), smem, stream, (const T*)rkv, ld, r_off, k_off, v_off, d_raw, \
               ldd, u, state, slots, token_req, req_first_token, o, ldo, H, K, V, VB, false)
#define WK_NS(T)                 \
  switch (NS) {                  \
    case 1: WK_GO(T, 1); break;  \
    case 2: WK_GO(T, 2); break;  \
    case 4: WK_GO(T, 4); break;  \
    case 8: WK_GO(T, 8); break;  \
    case 16: WK_GO(T, 16); break; \
    default: WK_GO(T, 32); break; \
  }
  if (dtype == MLXB_F32) { WK_NS(float) }
  else if (dtype == MLXB_BF16) { WK_NS(__nv_bfloat16) }
  else return mlxb_fail(MLXB_BAD_DTYPE, "wkv_scan: dtype code %d", dtype);
#undef WK_NS
#undef WK_GO
  return mlxb_check_launch("wkv_scan");
}
