// The attention of attention_wide.cu on tensor cores (mma.sync, bfloat16 pages, float32 accumulation).
//
// A CTA takes 32 rows: TQ consecutive tokens of one request times HG neighbouring heads that share a value head
// (TQ * HG = 32; a single-token entry: one token, HG heads, the other rows empty), and walks the keys in blocks of
// 64 positions that start at multiples of 64, so the order of additions for a row depends on its position only.
//
// Queries arrive in float32 and are used as two bfloat16 halves (hi + lo, two products per tile): nothing is
// lost of them.  Scores mixed across heads (talk [H, H]) are computed as products of MIXED QUERIES: with
// s'_h = sum_g talk[h, g] scale q_g . k_kv(g), grouping the heads g by their key head c gives
// s'_h = scale sum_c (sum_{g in c} talk[h, g] q_g) . k_c, an ordinary score of a query of G*dk dimensions against the
// token's G key heads laid side by side; the mixed query is made in float32 when the CTA loads its queries.
//
// Per block of keys: the K tile (and the V tile, unless the values are the first Dv columns of the key rows) comes
// into shared memory by 16-byte cp.async through the block table; warp w takes the scores of keys 8w .. 8w+7 for
// all 32 rows (S = Q K^T), masked and scaled into shared memory in float32; eight threads a row keep the running
// maximum and sum and write the weights as bfloat16; warp w then takes every eighth 8-column tile of the values
// (O = O * corr + P V) in registers.  Masks: causal, a window, runs of `chunk` positions counted from 0.
#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

constexpr int TC_M = 32, TC_N = 64, TC_THREADS = 256, TC_WARPS = 8;
constexpr int TC_NT = 8;      // 8-column value tiles a warp accumulates: Dv <= 8 * 8 * TC_NT = 512
constexpr int TC_SPAD = 4, TC_PPAD = 8;

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned (&r)[2], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(unsigned (&r)[2], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory"); }

// tiles: int32 [n_tiles, 4] = (first token row, queries, block-table row, first position); a CTA takes tokens
// sub*TQ .. of tile blockIdx.x / subs.  DkE: columns of a (mixed) query and of a key tile row, a multiple of 16;
// seg: columns one key head gives (talk: dk, G segments side by side; else Dk8 = the key's columns rounded up to 8,
// one segment).  shared_v: values are columns 0 .. Dv-1 of the key tile.
template <typename TO>
__global__ void __launch_bounds__(TC_THREADS, 2)
attention_wide_tc_kernel(const float* q, int ldq, int qhs, const int* __restrict__ tiles, int subs, int TQ, int HG,
                         const int* __restrict__ block_table, int max_pages, int n_pages, int page, int Hq, int Hkv,
                         int Dk, int Dv, int DkE, int seg, int n_seg, int krs, int vrs, int shared_v, int window,
                         int chunk, float scale, const float* __restrict__ talk, const __nv_bfloat16* k_pool,
                         const __nv_bfloat16* v_pool, const __nv_bfloat16* gate, int ldg, TO* __restrict__ out, int ldo,
                         int ohs, int* __restrict__ status, int bps, int n_rel, float* __restrict__ scratch) {
  extern __shared__ __align__(16) unsigned char tc_smem[];
  const int ldk = DkE + 8, ldv = shared_v ? ldk : Dv + 8;
  long long* sRow = reinterpret_cast<long long*>(tc_smem);                  // [TC_N]
  float* sS = reinterpret_cast<float*>(sRow + TC_N);                        // [TC_M][TC_N + TC_SPAD]
  float* sCorr = sS + TC_M * (TC_N + TC_SPAD);                              // [TC_M]
  float* sL = sCorr + TC_M;                                                 // [TC_M]
  __nv_bfloat16* sP = reinterpret_cast<__nv_bfloat16*>(sL + TC_M);          // [TC_M][TC_N + TC_PPAD]
  __nv_bfloat16* sQh = sP + TC_M * (TC_N + TC_PPAD);                        // [TC_M][ldk]
  __nv_bfloat16* sQl = sQh + TC_M * ldk;                                    // [TC_M][ldk]
  __nv_bfloat16* sK = sQl + TC_M * ldk;                                     // [TC_N][ldk]
  __nv_bfloat16* sV = shared_v ? sK : sK + TC_N * ldk;                      // [TC_N][ldv]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tile = blockIdx.x / subs, sub = blockIdx.x - tile * subs;
  const int t_first = tiles[4 * tile], n_tile = tiles[4 * tile + 1], bt_row = tiles[4 * tile + 2];
  const int nq = min(TQ, n_tile - sub * TQ);
  if (nq <= 0) return;
  const int t0 = t_first + sub * TQ, pos0 = tiles[4 * tile + 3] + sub * TQ;
  const int h0 = blockIdx.y * HG, rep = Hq / Hkv, cv = h0 / rep;
  const int* bt = block_table + (size_t)bt_row * max_pages;
  int lo_min = 0;                                            // first visible key of the first token: the smallest of the CTA
  if (window > 0 && pos0 - window + 1 > lo_min) lo_min = pos0 - window + 1;
  if (chunk > 0 && (pos0 / chunk) * chunk > lo_min) lo_min = (pos0 / chunk) * chunk;
  if (bps > 0 && ((lo_min / TC_N) / bps + (int)blockIdx.z) * bps * TC_N > pos0 + nq - 1) return;   // a split without keys
  pdl_wait();
  pdl_trigger();
  q = after_wait(q);
  k_pool = after_wait(k_pool);
  v_pool = after_wait(v_pool);
  gate = after_wait(gate);
  // ---- queries: float32 -> hi + lo; with talk, the heads' queries mixed into the key heads' segments
  const int rows_used = nq * HG;                             // rows 0 .. rows_used - 1 carry a (token, head)
  for (int e = tid; e < rows_used * DkE; e += TC_THREADS) {
    const int r = e / DkE, col = e - r * DkE;
    const int tq = r / HG, h = h0 + r % HG;
    float v = 0.f;
    const float* qt = q + (size_t)(t0 + tq) * ldq;
    if (talk) {
      const int c = col / seg, d = col - c * seg;
      if (c < n_seg)
        for (int i = 0; i < rep; ++i) v = fmaf(talk[h * Hq + c * rep + i], qt[(size_t)(c * rep + i) * qhs + d], v);
    } else if (col < Dk) {
      v = qt[(size_t)h * qhs + col];
    }
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    sQh[r * ldk + col] = hi;
    sQl[r * ldk + col] = __float2bfloat16_rn(v - __bfloat162float(hi));
  }
  for (int e = rows_used * (ldk / 8) + tid; e < TC_M * (ldk / 8); e += TC_THREADS) {      // the empty rows: zeros
    reinterpret_cast<uint4*>(sQh)[e] = make_uint4(0u, 0u, 0u, 0u);
    reinterpret_cast<uint4*>(sQl)[e] = make_uint4(0u, 0u, 0u, 0u);
  }
  // the rows' visible ranges
  const int my_row = tid >> 3, my_sub = tid & 7;             // softmax: eight threads a row
  const int my_tq = my_row / HG;
  const int my_p = my_tq < nq ? pos0 + my_tq : -1;
  int my_lo = 0;
  if (window > 0 && my_p - window + 1 > my_lo) my_lo = my_p - window + 1;
  if (chunk > 0 && (my_p / chunk) * chunk > my_lo) my_lo = (my_p / chunk) * chunk;
  int p_max = pos0 + nq - 1;
  int j_first = (lo_min / TC_N) * TC_N;
  if (bps > 0) {
    // single rows with their keys split over the CTAs of grid.z: this one takes the blocks bps*za .. bps*za + bps - 1,
    // counted from position 0, and leaves an unnormalised partial result for the merge kernel
    const int za = (lo_min / TC_N) / bps + blockIdx.z;
    j_first = max(j_first, za * bps * TC_N);
    p_max = min(p_max, (za + 1) * bps * TC_N - 1);
  }
  float m_run = -INFINITY, l_run = 0.f;
  float o[TC_NT][2][4];
#pragma unroll
  for (int i = 0; i < TC_NT; ++i)
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int x = 0; x < 4; ++x) o[i][m][x] = 0.f;
  const int n_vt = Dv / 8;                                   // 8-column tiles of the values
  const int g = lane >> 2, tq4 = lane & 3;

  for (int j0 = j_first; j0 <= p_max; j0 += TC_N) {
    __syncthreads();                                         // the block before is done with the tiles
    if (tid < TC_N) {
      const int j = j0 + tid;
      long long row = -1;
      if (j >= lo_min && j <= p_max) {
        const int lp = j / page;
        const int pg = lp < max_pages ? bt[lp] : -1;
        if (pg >= n_pages) atomicOr(status, MLXB_ST_PAGE_RANGE);
        else if (pg < 0) atomicOr(status, MLXB_ST_POSITION_RANGE);
        else row = (long long)pg * Hkv * page + (j % page);
      }
      sRow[tid] = row;
    }
    __syncthreads();
    {
      const int per_key = DkE / 8;                           // 16-byte pieces of a key tile row
      for (int e = tid; e < TC_N * per_key; e += TC_THREADS) {
        const int jj = e / per_key, col = (e - jj * per_key) * 8;
        const long long row = sRow[jj];
        __nv_bfloat16* dst = sK + jj * ldk + col;
        const int c = col / seg, d = col - c * seg;
        if (row >= 0 && c < n_seg && d < seg)
          cp_async16(dst, k_pool + (size_t)(row + (long long)(talk ? c : cv) * page) * krs + d);
        else
          *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
      }
      if (!shared_v) {
        const int per_v = Dv / 8;
        for (int e = tid; e < TC_N * per_v; e += TC_THREADS) {
          const int jj = e / per_v, col = (e - jj * per_v) * 8;
          const long long row = sRow[jj];
          __nv_bfloat16* dst = sV + jj * ldv + col;
          if (row >= 0) cp_async16(dst, v_pool + (size_t)(row + (long long)cv * page) * vrs + col);
          else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      cp_async_wait_all();
    }
    __syncthreads();
    // ---- S = Q K^T for keys 8 warp .. 8 warp + 7
    {
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const unsigned kb = smem_addr(sK + (warp * 8 + (lane & 7)) * ldk + ((lane >> 3) & 1) * 8);
      const unsigned qh = smem_addr(sQh + (lane & 15) * ldk + (lane >> 4) * 8);
      const unsigned ql = smem_addr(sQl + (lane & 15) * ldk + (lane >> 4) * 8);
      for (int k0 = 0; k0 < DkE; k0 += 16) {
        unsigned b[2], a[4];
        ldmatrix_x2(b, kb + k0 * 2);
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          ldmatrix_x4(a, qh + (m * 16 * ldk + k0) * 2);
          mma_bf16(s[m], a, b);
          ldmatrix_x4(a, ql + (m * 16 * ldk + k0) * 2);
          mma_bf16(s[m], a, b);
        }
      }
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const int r = m * 16 + g + (x >> 1) * 8, jj = warp * 8 + tq4 * 2 + (x & 1);
          sS[r * (TC_N + TC_SPAD) + jj] = s[m][x] * scale;
        }
    }
    __syncthreads();
    // ---- weights: eight threads a row, eight keys each
    {
      float sv[8];
      float mb = -INFINITY;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int jj = my_sub * 8 + i, j = j0 + jj;
        const bool vis = j <= my_p && j >= my_lo && sRow[jj] >= 0;
        sv[i] = vis ? sS[my_row * (TC_N + TC_SPAD) + jj] : -INFINITY;
        mb = fmaxf(mb, sv[i]);
      }
      mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 1));
      mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 2));
      mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 4));
      const float m_new = fmaxf(m_run, mb);
      const float corr = m_run == -INFINITY ? 0.f : expf(m_run - m_new);
      float sum = 0.f;
      __nv_bfloat16* pr = sP + my_row * (TC_N + TC_PPAD) + my_sub * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float pw = sv[i] == -INFINITY ? 0.f : expf(sv[i] - m_new);
        const __nv_bfloat16 pb = __float2bfloat16_rn(pw);
        pr[i] = pb;
        sum += __bfloat162float(pb);                         // the sum of what the values are weighted with
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      l_run = l_run * corr + sum;
      m_run = m_new;
      if (my_sub == 0) sCorr[my_row] = corr;
    }
    __syncthreads();
    // ---- O = O corr + P V for this warp's value tiles
    {
      float cr[2][2];
#pragma unroll
      for (int m = 0; m < 2; ++m) { cr[m][0] = sCorr[m * 16 + g]; cr[m][1] = sCorr[m * 16 + g + 8]; }
      unsigned a[2][4][4];                                   // P: two row tiles x four key steps
      const unsigned pb = smem_addr(sP + (lane & 15) * (TC_N + TC_PPAD) + (lane >> 4) * 8);
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) ldmatrix_x4(a[m][ks], pb + (m * 16 * (TC_N + TC_PPAD) + ks * 16) * 2);
#pragma unroll
      for (int i = 0; i < TC_NT; ++i) {
        const int nt = warp + i * TC_WARPS;
        if (nt < n_vt) {
#pragma unroll
          for (int m = 0; m < 2; ++m) {
            o[i][m][0] *= cr[m][0]; o[i][m][1] *= cr[m][0];
            o[i][m][2] *= cr[m][1]; o[i][m][3] *= cr[m][1];
          }
          const unsigned vb = smem_addr(sV + (lane & 15) * ldv + nt * 8);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            unsigned b[2];
            ldmatrix_x2_trans(b, vb + ks * 16 * ldv * 2);
            mma_bf16(o[i][0], a[0][ks], b);
            mma_bf16(o[i][1], a[1][ks], b);
          }
        }
      }
    }
  }
  if (my_sub == 0) sL[my_row] = l_run;
  __syncthreads();
  if (bps > 0) {
    // partial results (TQ = 1: row r is head h0 + r): [tile, head, split][Dv values | maximum | sum]
    const size_t stride = (size_t)Dv + 2;
    if (my_sub == 0 && my_row < HG) {
      float* sp = scratch + (((size_t)tile * Hq + h0 + my_row) * n_rel + blockIdx.z) * stride;
      sp[Dv] = m_run;
      sp[Dv + 1] = l_run;
    }
#pragma unroll
    for (int i = 0; i < TC_NT; ++i) {
      const int nt = warp + i * TC_WARPS;
      if (nt >= n_vt) continue;
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = m * 16 + g + half * 8;
          if (r >= HG) continue;
          float* sp = scratch + (((size_t)tile * Hq + h0 + r) * n_rel + blockIdx.z) * stride + nt * 8 + tq4 * 2;
          sp[0] = o[i][m][half * 2];
          sp[1] = o[i][m][half * 2 + 1];
        }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < TC_NT; ++i) {
    const int nt = warp + i * TC_WARPS;
    if (nt >= n_vt) continue;
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = m * 16 + g + half * 8;
        const int tq = r / HG, h = h0 + r % HG;
        if (tq >= nq) continue;
        const float l = sL[r];
        float f = l > 0.f ? 1.f / l : 0.f;
        const int t = t0 + tq;
        if (gate) f *= 1.f / (1.f + expf(-__bfloat162float(gate[(size_t)t * ldg + h])));
        TO* op = out + (size_t)t * ldo + (size_t)h * ohs + nt * 8 + tq4 * 2;
        op[0] = from_f<TO>(o[i][m][half * 2] * f);
        op[1] = from_f<TO>(o[i][m][half * 2 + 1] * f);
      }
  }
}

// The partial results of a single row's splits, merged in the order of the splits: one block per (tile, head).
template <typename TO>
__global__ void attention_wide_merge_kernel(const int* __restrict__ tiles, int Hq, int Dv, int window, int chunk, int bps,
                                            int n_rel, const float* scratch, const __nv_bfloat16* gate, int ldg,
                                            TO* __restrict__ out, int ldo, int ohs) {
  const int tile = blockIdx.x, h = blockIdx.y;
  if (tiles[4 * tile + 1] <= 0) return;
  const int t = tiles[4 * tile], p = tiles[4 * tile + 3];
  int lo = 0;
  if (window > 0 && p - window + 1 > lo) lo = p - window + 1;
  if (chunk > 0 && (p / chunk) * chunk > lo) lo = (p / chunk) * chunk;
  const int nz = (p / TC_N) / bps - (lo / TC_N) / bps + 1;
  pdl_wait();
  pdl_trigger();
  scratch = after_wait(scratch);
  gate = after_wait(gate);
  const size_t stride = (size_t)Dv + 2;
  const float* sp = scratch + ((size_t)tile * Hq + h) * n_rel * stride;
  float M = -INFINITY;
  for (int z = 0; z < nz; ++z) M = fmaxf(M, sp[z * stride + Dv]);
  float L = 0.f;
  for (int z = 0; z < nz; ++z) {
    const float mz = sp[z * stride + Dv];
    if (mz != -INFINITY) L = fmaf(expf(mz - M), sp[z * stride + Dv + 1], L);
  }
  float f = L > 0.f ? 1.f / L : 0.f;
  if (gate) f *= 1.f / (1.f + expf(-__bfloat162float(gate[(size_t)t * ldg + h])));
  for (int c = threadIdx.x; c < Dv; c += blockDim.x) {
    float a = 0.f;
    for (int z = 0; z < nz; ++z) {
      const float mz = sp[z * stride + Dv];
      if (mz != -INFINITY) a = fmaf(expf(mz - M), sp[z * stride + c], a);
    }
    out[(size_t)t * ldo + (size_t)h * ohs + c] = from_f<TO>(a * f);
  }
}

constexpr int TC_BPS = 2;     // key blocks a CTA of a split single row takes: a constant, never a function of the batch

// Splits a single row can have: the positions it can see, in blocks, over TC_BPS, and one more at either end.
static int tc_splits(int window, int chunk, int max_len) {
  int span = max_len > 0 ? max_len : 1;
  if (window > 0 && window < span) span = window;
  if (chunk > 0 && chunk < span) span = chunk;
  return ((span + TC_N - 1) / TC_N + 1) / TC_BPS + 2;
}

// Floats of scratch memory that single rows need (0: rows that see at most two blocks are not split).
MLXB_EXPORT long long mlxb_attention_wide_tc_scratch(int n_rows, int Hq, int Dv, int window, int chunk, int max_len) {
  const int n_rel = tc_splits(window, chunk, max_len);
  if (n_rel <= 3) return 0;
  return (long long)n_rows * Hq * n_rel * (Dv + 2);
}

// What the launch needs of shared memory, or -1 if the sizes are not served (the caller then takes the kernel on the
// CUDA cores): key and value widths in whole 16-byte pieces, at most 512 value columns, heads that group.
static long long tc_plan(int Hq, int Hkv, int Dk, int Dv, int krs, int vrs, int talk, int shared_v, int* DkE, int* seg,
                         int* n_seg, int* HG) {
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || Dv % 8 || Dv > 64 * TC_NT || krs % 8 || vrs % 8) return -1;
  const int rep = Hq / Hkv;
  if (talk) {
    if (Dk % 8) return -1;
    *seg = Dk;
    *n_seg = Hkv;
  } else {
    *seg = (Dk + 7) / 8 * 8;          // the pool's rows are zero beyond Dk
    if (*seg > krs) return -1;
    *n_seg = 1;
  }
  *DkE = ((*seg) * (*n_seg) + 15) / 16 * 16;
  if (shared_v && Dv > *DkE) return -1;
  int hg = 1;
  while (hg * 2 <= TC_M && rep % (hg * 2) == 0) hg *= 2;
  *HG = hg;
  const int ldk = *DkE + 8, ldv = shared_v ? ldk : Dv + 8;
  const long long bytes = 8LL * TC_N + 4LL * (TC_M * (TC_N + TC_SPAD) + 2 * TC_M) + 2LL * TC_M * (TC_N + TC_PPAD) +
                          2LL * (2 * TC_M + TC_N) * ldk + (shared_v ? 0LL : 2LL * TC_N * ldv);
  return bytes <= 200 * 1024 ? bytes : -1;
}

MLXB_EXPORT int mlxb_attention_wide_tc_supported(int Hq, int Hkv, int Dk, int Dv, int krs, int vrs, int talk, int shared_v) {
  int a, b, c, d;
  return tc_plan(Hq, Hkv, Dk, Dv, krs, vrs, talk, shared_v, &a, &b, &c, &d) >= 0;
}

// The arguments of mlxb_attention_wide with bfloat16 pools, and instead of the token rows a list of tiles: int32
// [n_tiles, 4] = (first token row, queries, block-table row, first position), each of at most tile_q queries.
MLXB_EXPORT int mlxb_attention_wide_tc(int out_f32, const float* q, int ldq, int qhs, const int* tiles, int n_tiles,
                                       int tile_q, const int* block_table, int max_pages, int n_pages, int page, int Hq,
                                       int Hkv, int Dk, int Dv, int krs, int vrs, int window, int chunk, float scale,
                                       const float* talk, const void* k_pool, const void* v_pool, const void* gate,
                                       int ldg, void* out, int ldo, int ohs, int* status, float* scratch, int max_len,
                                       cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  int DkE, seg, n_seg, HG;
  const int shared_v = v_pool == k_pool;
  const long long smem = tc_plan(Hq, Hkv, Dk, Dv, krs, vrs, talk != nullptr, shared_v, &DkE, &seg, &n_seg, &HG);
  if (smem < 0 || page <= 0 || (page & (page - 1)) || tile_q <= 0 || qhs < Dk || ohs < Dv)
    return mlxb_fail(MLXB_BAD_ARG, "attention (wide, tensor cores): %d/%d heads, sizes %d/%d in rows of %d/%d", Hq, Hkv,
                     Dk, Dv, krs, vrs);
  // single rows with scratch memory: their keys split over grid.z, then merged
  const int n_rel = tc_splits(window, chunk, max_len);
  const bool split = tile_q == 1 && scratch != nullptr && n_rel > 3;
  const int TQ = split ? 1 : TC_M / HG;
  const int subs = (tile_q + TQ - 1) / TQ;
  const int bps = split ? TC_BPS : 0;
  const dim3 grid((unsigned)n_tiles * subs, Hq / HG, split ? n_rel : 1), block(TC_THREADS);
#define TCW_GO(TO)                                                                                                     \
  do {                                                                                                                 \
    auto kern = attention_wide_tc_kernel<TO>;                                                                          \
    if (smem > 48 * 1024) {                                                                                            \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
      if (e != cudaSuccess)                                                                                            \
        return mlxb_fail((int)e, "attention (wide, tensor cores): %lld bytes of shared memory: %s", smem,              \
                         cudaGetErrorString(e));                                                                       \
    }                                                                                                                  \
    launch_pdl(kern, grid, block, (size_t)smem, stream, q, ldq, qhs, tiles, subs, TQ, HG, block_table, max_pages,      \
               n_pages, page, Hq, Hkv, Dk, Dv, DkE, seg, n_seg, krs, vrs, shared_v, window, chunk, scale, talk,        \
               (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, (const __nv_bfloat16*)gate, ldg, (TO*)out,  \
               ldo, ohs, status, bps, n_rel, scratch);                                                                 \
    if (split) {                                                                                                       \
      if (int e = mlxb_check_launch("attention (wide, tensor cores)")) return e;                                       \
      launch_pdl(attention_wide_merge_kernel<TO>, dim3(n_tiles, Hq), dim3(Dv >= 128 ? 128 : 64), 0, stream, tiles, Hq, \
                 Dv, window, chunk, bps, n_rel, (const float*)scratch, (const __nv_bfloat16*)gate, ldg, (TO*)out, ldo, \
                 ohs);                                                                                                 \
    }                                                                                                                  \
  } while (0)
  if (out_f32) TCW_GO(float);
  else TCW_GO(__nv_bfloat16);
#undef TCW_GO
  return mlxb_check_launch("attention (wide, tensor cores)");
}
