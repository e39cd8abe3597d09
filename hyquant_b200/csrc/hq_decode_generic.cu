// Decode attention over the four-segment cache for the bit widths other than K4/V4
// (K or V prefix in 8, 4 or 2 bits; reference src/ops/decode_d_stage.py:270-1005 covers them with one
// Triton kernel family).  A plain CUDA-core kernel: the K4/V4 path, which the benchmarks run, has its own
// tensor-core kernel in hq_decode.cu.
//
// HBM bytes per call: BH_KV * ((16 KB + 16 VB + 4) * n_quant + 512 * (n_topk + n_staging + n_window)) + 512 * BH_Q
// with KB / VB the bit widths (a token row is 16 * bits bytes).
//
// Work decomposition.  The tokens of a head's four segments are cut into chunks of 32 tokens; a CTA owns a
// contiguous range of one head's chunks, its 8 warps take them round-robin.  Per chunk: lane = token for the
// scores (each lane reads its token's K row with 16-byte loads and dots it with the group's query rows,
// which sit in shared memory as fp32), one online-softmax step in base 2 for the 32 tokens, then lane =
// 4 channels for P V (every lane reads its 4 channels of each token's V row — all of a chunk's V loads are issued
// before the score phase so that they are in flight during it — and the token's probabilities come by shuffle).  Warps and then CTAs merge through the log-sum-exp rule; the splits of a head are merged
// by a second, tiny kernel (lse_merge_kernel of hq_reorg.cu).
#include "hq_common.cuh"

namespace hq {

struct GenericParams {
  const __nv_bfloat16* q; int64_t q_stride;
  const uint8_t* k_packed; const uint8_t* v_packed; int64_t kp_stride_bh, vp_stride_bh;
  const __half* k_scale; const __half* v_scale; int64_t ks_stride_bh, vs_stride_bh;
  const __nv_bfloat16* kseg[3]; const __nv_bfloat16* vseg[3]; int64_t kseg_stride[3], vseg_stride[3];
  int nseg[4];                 // tokens: quantised prefix, topk, staging, window
  int cseg[4];                 // chunks of 32 tokens per segment
  int chunks;                  // total
  int nsplit, R;
  float sml;                   // sm_scale * log2(e)
  float* ws_m; float* ws_l; float* ws_acc;     // [nsplit][BH_Q], [nsplit][BH_Q], [nsplit][BH_Q][128]
  int64_t rows;                // BH_Q
};

constexpr int kGWarps = 8;

// codes of `bits` width in a little-endian word -> sign-extended ints
template <int BITS>
__device__ __forceinline__ int code_at(uint32_t w, int i) {
  return ((int)(w << (32 - BITS * (i + 1)))) >> (32 - BITS);
}

// dot products of one token's quantised K row (16 * BITS bytes) with RMAX query rows in shared memory
template <int BITS, int RMAX>
__device__ __forceinline__ void k_dot_quant(const uint8_t* row, const float* qs, int R, float (&s)[RMAX]) {
  constexpr int kWords = 4 * BITS;                 // 32-bit words per row
  constexpr int kPerWord = 32 / BITS;              // codes per word: 4, 8 or 16 consecutive channels
#pragma unroll
  for (int w4 = 0; w4 < kWords / 4; ++w4) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(row) + w4);
    const uint32_t ws[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
      for (int i4 = 0; i4 < kPerWord / 4; ++i4) {
        const int c = (w4 * 4 + wi) * kPerWord + 4 * i4;       // 4 channels, one 16-byte read of each query row
        const float x0 = (float)code_at<BITS>(ws[wi], 4 * i4), x1 = (float)code_at<BITS>(ws[wi], 4 * i4 + 1);
        const float x2 = (float)code_at<BITS>(ws[wi], 4 * i4 + 2), x3 = (float)code_at<BITS>(ws[wi], 4 * i4 + 3);
#pragma unroll
        for (int h = 0; h < RMAX; ++h) {
          if (h < R) {
            const float4 qv = *reinterpret_cast<const float4*>(qs + h * 128 + c);
            s[h] = fmaf(x3, qv.w, fmaf(x2, qv.z, fmaf(x1, qv.y, fmaf(x0, qv.x, s[h]))));
          }
        }
      }
    }
  }
}

template <int RMAX>
__device__ __forceinline__ void k_dot_bf16(const __nv_bfloat16* row, const float* qs, int R, float (&s)[RMAX]) {
#pragma unroll 4
  for (int w4 = 0; w4 < 16; ++w4) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(row) + w4);
    const float x[8] = {__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u), __uint_as_float(u.y << 16),
                        __uint_as_float(u.y & 0xFFFF0000u), __uint_as_float(u.z << 16), __uint_as_float(u.z & 0xFFFF0000u),
                        __uint_as_float(u.w << 16), __uint_as_float(u.w & 0xFFFF0000u)};
#pragma unroll
    for (int h = 0; h < RMAX; ++h) {
      if (h < R) {
        const float4 qa = *reinterpret_cast<const float4*>(qs + h * 128 + 8 * w4);
        const float4 qb = *reinterpret_cast<const float4*>(qs + h * 128 + 8 * w4 + 4);
        s[h] = fmaf(x[3], qa.w, fmaf(x[2], qa.z, fmaf(x[1], qa.y, fmaf(x[0], qa.x, s[h]))));
        s[h] = fmaf(x[7], qb.w, fmaf(x[6], qb.z, fmaf(x[5], qb.y, fmaf(x[4], qb.x, s[h]))));
      }
    }
  }
}

template <int KB, int VB, int RMAX>
__global__ void __launch_bounds__(kGWarps * 32)
decode_generic_kernel(const GenericParams p) {
  __shared__ __align__(16) float qs[RMAX * 128];
  __shared__ float mrg_m[kGWarps][RMAX], mrg_l[kGWarps][RMAX];
  extern __shared__ float mrg_acc[];             // [kGWarps][R][128]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int head = blockIdx.y, split = blockIdx.x, R = p.R;
  for (int x = tid; x < R * 128; x += blockDim.x)
    qs[x] = __bfloat162float(p.q[(int64_t)(head * R + (x >> 7)) * p.q_stride + (x & 127)]);
  __syncthreads();

  float m[RMAX], l[RMAX], acc[RMAX][4];
#pragma unroll
  for (int h = 0; h < RMAX; ++h) {
    m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[h][c] = 0.f;
  }
  const int c_begin = (int)(((int64_t)split * p.chunks) / p.nsplit);
  const int c_end = (int)(((int64_t)(split + 1) * p.chunks) / p.nsplit);
  for (int ch = c_begin + warp; ch < c_end; ch += kGWarps) {
    int seg = 0, cc = ch;
    while (seg < 3 && cc >= p.cseg[seg]) { cc -= p.cseg[seg]; ++seg; }
    const int tok0 = cc * 32, ntok = min(32, p.nseg[seg] - tok0);
    const int tok = tok0 + lane;
    const bool ok = lane < ntok;
    // ---- the chunk's V words first (this lane's 4 channels of every token, coalesced rows): all of them are in
    // flight while the scores are computed.  BF16 rows are 8 bytes per lane and token and come in two halves.
    uint32_t vw[32];
    const uint8_t* vrow0 = nullptr;
    const uint2* vrow2 = nullptr;
    if (seg == 0) {
      vrow0 = p.v_packed + head * p.vp_stride_bh + (int64_t)tok0 * (16 * VB);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        vw[j] = 0u;
        if (j < ntok) {
          const uint8_t* row = vrow0 + (int64_t)j * (16 * VB);
          if (VB == 8) vw[j] = __ldg(reinterpret_cast<const uint32_t*>(row) + lane);
          else if (VB == 4) vw[j] = __ldg(reinterpret_cast<const uint16_t*>(row) + lane);
          else vw[j] = __ldg(row + lane);
        }
      }
    } else {
      vrow2 = reinterpret_cast<const uint2*>(p.vseg[seg - 1] + head * p.vseg_stride[seg - 1] + (int64_t)tok0 * 128) + lane;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        uint2 u = make_uint2(0u, 0u);
        if (j < ntok) u = __ldg(vrow2 + j * 32);
        vw[2 * j] = u.x; vw[2 * j + 1] = u.y;
      }
    }
    // ---- scores of this lane's token against the group's heads
    float s[RMAX];
#pragma unroll
    for (int h = 0; h < RMAX; ++h) s[h] = 0.f;
    float vscale = 0.f;
    if (ok) {
      if (seg == 0) {
        k_dot_quant<KB, RMAX>(p.k_packed + head * p.kp_stride_bh + (int64_t)tok * (16 * KB), qs, R, s);
        const float ksc = __half2float(p.k_scale[head * p.ks_stride_bh + tok]) * p.sml;
        vscale = __half2float(p.v_scale[head * p.vs_stride_bh + tok]);
#pragma unroll
        for (int h = 0; h < RMAX; ++h) s[h] *= ksc;
      } else {
        k_dot_bf16<RMAX>(p.kseg[seg - 1] + head * p.kseg_stride[seg - 1] + (int64_t)tok * 128, qs, R, s);
        vscale = 1.f;
#pragma unroll
        for (int h = 0; h < RMAX; ++h) s[h] *= p.sml;
      }
    }
    // ---- one online-softmax step for the chunk
    float pr[RMAX];
#pragma unroll
    for (int h = 0; h < RMAX; ++h) {
      float mx = ok ? s[h] : -INFINITY;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float nm = fmaxf(m[h], mx);
      const float alpha = (nm == -INFINITY) ? 1.f : ex2f(m[h] - nm);      // m = -inf -> 0
      m[h] = nm;
      pr[h] = ok ? ex2f(s[h] - nm) : 0.f;
      l[h] = l[h] * alpha + pr[h];                                        // lane-local part of the row sum
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[h][c] *= alpha;
      pr[h] *= vscale;                                                     // the token's V scale rides in P
    }
    // ---- P V: this lane owns channels 4 lane .. 4 lane + 3
    if (seg == 0) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = (float)code_at<VB>(vw[j], i);
#pragma unroll
        for (int h = 0; h < RMAX; ++h) {
          if (h < R) {
            const float pj = __shfl_sync(0xffffffffu, pr[h], j);       // 0 for tokens past ntok
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[h][c] = fmaf(pj, v[c], acc[h][c]);
          }
        }
      }
    } else {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if (half == 1) {
          if (ntok <= 16) break;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            uint2 u = make_uint2(0u, 0u);
            if (16 + j < ntok) u = __ldg(vrow2 + (16 + j) * 32);
            vw[2 * j] = u.x; vw[2 * j + 1] = u.y;
          }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float v[4] = {__uint_as_float(vw[2 * j] << 16), __uint_as_float(vw[2 * j] & 0xFFFF0000u),
                              __uint_as_float(vw[2 * j + 1] << 16), __uint_as_float(vw[2 * j + 1] & 0xFFFF0000u)};
#pragma unroll
          for (int h = 0; h < RMAX; ++h) {
            if (h < R) {
              const float pj = __shfl_sync(0xffffffffu, pr[h], 16 * half + j);
#pragma unroll
              for (int c = 0; c < 4; ++c) acc[h][c] = fmaf(pj, v[c], acc[h][c]);
            }
          }
        }
      }
    }
  }
  // ---- merge the warps, write this split's partial
#pragma unroll
  for (int h = 0; h < RMAX; ++h) {
    float ls = l[h];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o);
    if (h < R) {
      if (lane == 0) { mrg_m[warp][h] = m[h]; mrg_l[warp][h] = ls; }
      *reinterpret_cast<float4*>(mrg_acc + ((size_t)(warp * R + h)) * 128 + 4 * lane) =
          make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
    }
  }
  __syncthreads();
  const int d = tid & 127;
  for (int h = tid >> 7; h < R; h += (kGWarps * 32) / 128) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kGWarps; ++w) M = fmaxf(M, mrg_m[w][h]);
    float a = 0.f, ls = 0.f;
#pragma unroll
    for (int w = 0; w < kGWarps; ++w) {
      const float mw = mrg_m[w][h];
      const float wt = (mw == -INFINITY) ? 0.f : ex2f(mw - M);
      a += wt * mrg_acc[((size_t)(w * R + h)) * 128 + d];
      ls += wt * mrg_l[w][h];
    }
    const int64_t prow = (int64_t)split * p.rows + (int64_t)head * R + h;
    p.ws_acc[prow * 128 + d] = a;
    if (d == 0) { p.ws_m[prow] = M; p.ws_l[prow] = ls; }
  }
}

template <int KB, int VB>
static int launch_generic_r(const GenericParams& p, dim3 grid, cudaStream_t st) {
  const size_t smem = (size_t)kGWarps * p.R * 128 * sizeof(float);     // <= 64 KB at R = 16
  if (p.R <= 4) {
    decode_generic_kernel<KB, VB, 4><<<grid, kGWarps * 32, smem, st>>>(p);
  } else if (p.R <= 8) {
    decode_generic_kernel<KB, VB, 8><<<grid, kGWarps * 32, smem, st>>>(p);
  } else {
    static thread_local int attr_dev = -1;
    int dev = 0;
    HQ_CUDA(cudaGetDevice(&dev));
    if (attr_dev != dev) {
      HQ_CUDA(cudaFuncSetAttribute(decode_generic_kernel<KB, VB, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536));
      attr_dev = dev;
    }
    decode_generic_kernel<KB, VB, 16><<<grid, kGWarps * 32, smem, st>>>(p);
  }
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}

template <int KB>
static int launch_generic_v(const GenericParams& p, int v_bits, dim3 grid, cudaStream_t st) {
  if (v_bits == 8) return launch_generic_r<KB, 8>(p, grid, st);
  if (v_bits == 4) return launch_generic_r<KB, 4>(p, grid, st);
  return launch_generic_r<KB, 2>(p, grid, st);
}

// Called by hq_decode_splitk for bit widths other than K4/V4, with its arguments already checked.
int decode_generic_launch(const hq_decode_args* a, int k_bits, int v_bits, float* ws, int64_t ws_floats, cudaStream_t st) {
  GenericParams p{};
  p.q = (const __nv_bfloat16*)a->q; p.q_stride = a->q_stride;
  p.k_packed = (const uint8_t*)a->k_packed; p.v_packed = (const uint8_t*)a->v_packed;
  p.kp_stride_bh = a->kp_stride_bh; p.vp_stride_bh = a->vp_stride_bh;
  p.k_scale = (const __half*)a->k_scale; p.v_scale = (const __half*)a->v_scale;
  p.ks_stride_bh = a->ks_stride_bh; p.vs_stride_bh = a->vs_stride_bh;
  const void* ks[3] = {a->k_topk, a->k_staging, a->k_window};
  const void* vs[3] = {a->v_topk, a->v_staging, a->v_window};
  const int64_t kst[3] = {a->kt_stride_bh, a->kg_stride_bh, a->kw_stride_bh};
  const int64_t vst[3] = {a->vt_stride_bh, a->vg_stride_bh, a->vw_stride_bh};
  const int ns[4] = {a->n_quant, a->n_topk, a->n_staging, a->n_window};
  p.chunks = 0;
  for (int s = 0; s < 4; ++s) {
    p.nseg[s] = ns[s];
    p.cseg[s] = (ns[s] + 31) / 32;
    p.chunks += p.cseg[s];
    if (s > 0) {
      p.kseg[s - 1] = (const __nv_bfloat16*)ks[s - 1]; p.vseg[s - 1] = (const __nv_bfloat16*)vs[s - 1];
      p.kseg_stride[s - 1] = kst[s - 1]; p.vseg_stride[s - 1] = vst[s - 1];
    }
  }
  HQ_REQUIRE(a->n_quant == 0 || (aligned16(a->k_packed) && a->kp_stride_bh % 16 == 0 && ((uintptr_t)a->v_packed % 4) == 0 &&
                                  a->vp_stride_bh % 4 == 0),
             HQ_ERR_ALIGNMENT, "hq_decode_splitk: packed K rows must be 16-byte aligned, packed V rows 4-byte aligned");
  p.R = a->kv_repeat;
  p.sml = a->sm_scale * 1.44269504f;
  p.rows = (int64_t)a->BH_KV * a->kv_repeat;
  // splits: about four CTAs per SM in all (the kernel hides its load latency with resident warps, not with a
  // prefetch ring), at least one chunk per warp, and the partials must fit the workspace
  int nsplit = a->num_splits > 0 ? a->num_splits : (4 * sm_count()) / a->BH_KV;
  const int by_work = (p.chunks + kGWarps - 1) / kGWarps;
  if (nsplit > by_work) nsplit = by_work;
  const int64_t by_ws = ws_floats / (p.rows * 130);
  if (nsplit > by_ws) nsplit = (int)by_ws;
  if (nsplit < 1) nsplit = 1;
  HQ_REQUIRE(by_ws >= 1, HQ_ERR_WORKSPACE, "hq_decode_splitk: workspace too small for one partial per query row");
  p.nsplit = nsplit;
  p.ws_m = ws; p.ws_l = ws + (int64_t)nsplit * p.rows; p.ws_acc = ws + 2 * (int64_t)nsplit * p.rows;
  p.ws_acc = (float*)(((uintptr_t)p.ws_acc + 15) & ~(uintptr_t)15);
  dim3 grid((unsigned)nsplit, (unsigned)a->BH_KV);
  int rc;
  if (k_bits == 8) rc = launch_generic_v<8>(p, v_bits, grid, st);
  else if (k_bits == 4) rc = launch_generic_v<4>(p, v_bits, grid, st);
  else rc = launch_generic_v<2>(p, v_bits, grid, st);
  if (rc != HQ_OK) return rc;
  // merge the splits: normalised output, or the un-normalised state in partial mode
  if (a->partial_acc != nullptr)
    return hq_lse_merge_partial(p.ws_m, p.ws_l, p.ws_acc, p.rows, p.rows, p.rows * 128, nsplit, (int)p.rows, a->partial_m,
                                a->partial_l, a->partial_acc, st);
  return hq_lse_merge_strided(p.ws_m, p.ws_l, p.ws_acc, p.rows, p.rows, p.rows * 128, nsplit, (int)p.rows, a->out, a->out_dtype,
                              a->out_stride, st);
}

}  // namespace hq
