// Hybrid-precision causal prefill attention, GQA-native: entry points and vertical-line bookkeeping.
//
// For the 128-query block starting at s of query head h (kv head h / R):
//   keys j <  wla(s)          : INT8 QK^T (one scale per query row and per key row, smoothed K)
//                               unless j is a vertical line of head h -> masked there and taken
//                               from the gathered BF16 vertical tiles instead;
//   vertical lines < wla(s)   : BF16 QK^T on the gathered rows (ascending position);
//   keys in [wla(s), s + 128) : BF16 QK^T with the causal mask (local window + diagonal);
// with wla(s) = floor(max(0, s - (W - 1)) / 64) * 64 — the block rule of the reference kernel
// (src/ops/sage_unified.py:483-485, 538-544).  All tiles share one online softmax in base 2 and one
// fp32 accumulator; P V runs in BF16.  Unlike the reference nothing is expanded to query heads or
// physically reordered: K / V stay at kv-head granularity and a per (query head, key) additive
// term of the INT8 score conversion, -inf on the head's vertical lines, removes those columns from
// the INT8 pass.
//
// Tensor-bound.  FLOPs per call: 4 * B * H_Q * 128 * N (N + 1) / 2.  The attention kernel itself
// (tcgen05 / tensor memory / TMA) lives in hq_prefill_tc.cu.
#include "hq_common.cuh"

namespace hq {

// Vertical-line bookkeeping: for every (batch, query head) the ascending index list gives
//   k_bias[key]  = -12582912 * k_scale[key], or -inf if the key is a vertical line of this head: the
//                  INT8 pass turns an s32 score i into float as bits(i + 0x4B400000) = 12582912 + i and
//                  applies the key scale and this term in one fused multiply-add;
//   nv_valid[qb] = number of vertical lines below wla(128 qb)
// (the role of the reference's reorder_kv_for_vertical counts, src/ops/sage_unified.py:537-544)
__global__ void vertical_meta_kernel(const int* __restrict__ vasc, int T, int N, int Npad, int W, int nqb, int R,
                                     const float* __restrict__ k_scale, float* __restrict__ k_bias,
                                     int* __restrict__ nv_valid) {
  const int64_t bh = blockIdx.x;
  const float* ks = k_scale + (bh / R) * Npad;           // (b, hq) -> (b, hq / R): heads of a batch are contiguous
  float* kb = k_bias + bh * Npad;
  for (int x = threadIdx.x; x < Npad; x += blockDim.x) kb[x] = -12582912.0f * ks[x];
  if (T == 0) return;
  __syncthreads();
  const int* a = vasc + bh * T;
  for (int x = threadIdx.x; x < T; x += blockDim.x) {
    const int key = a[x];
    if (key >= 0 && key < N) kb[key] = -INFINITY;
  }
  for (int qb = threadIdx.x; qb < nqb; qb += blockDim.x) {
    const int s0 = qb * 128;
    const int wla = W > 0 ? (max(0, s0 - (W - 1)) / 64) * 64 : s0;
    int lo = 0, hi = T;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (a[mid] < wla) lo = mid + 1; else hi = mid; }
    nv_valid[bh * nqb + qb] = lo;
  }
}

}  // namespace hq

namespace hq {
int prefill_tc_launch(const hq_prefill_args* a, cudaStream_t st);
int prefill_tc_prepare_v(const void* v, int64_t sb, int64_t sh, int64_t sn, int B, int H_KV, int N, void* v_t, cudaStream_t st);
int prefill_tc_prepare_vertical(const int32_t* vasc, int B, int H_Q, int H_KV, int N, int T, const void* k_bf, const void* v,
                                int64_t v_sb, int64_t v_sh, int64_t v_sn, void* xk, void* xvt, cudaStream_t st);
int prefill_tc_prepare_v_fp8(const void* v, int64_t sb, int64_t sh, int64_t sn, int B, int H_KV, int N, void* v_t8, float* v_scale,
                             void* amax_scratch, cudaStream_t st);
int prefill_tc_gather_v_fp8(const int32_t* vasc, int B, int H_Q, int H_KV, int N, int T, const void* v, int64_t v_sb, int64_t v_sh,
                            int64_t v_sn, const float* v_scale, void* xvt8, cudaStream_t st);
}

extern "C" int hq_prefill_vertical_gather_v_fp8(const int32_t* vidx_asc, int B, int H_Q, int H_KV, int N, int T, const void* v,
                                                int64_t v_sb, int64_t v_sh, int64_t v_sn, const float* v_scale, void* vert_vt8,
                                                void* stream) {
  using namespace hq;
  HQ_REQUIRE(vidx_asc && v && v_scale && vert_vt8 && B > 0 && H_Q > 0 && H_KV > 0 && N > 0 && T > 0 && H_Q % H_KV == 0, HQ_ERR_INVALID,
             "hq_prefill_vertical_gather_v_fp8: bad arguments");
  HQ_REQUIRE(aligned16(v) && aligned16(vert_vt8) && v_sb % 8 == 0 && v_sh % 8 == 0 && v_sn % 8 == 0, HQ_ERR_ALIGNMENT,
             "hq_prefill_vertical_gather_v_fp8: rows must be 16-byte aligned");
  return prefill_tc_gather_v_fp8(vidx_asc, B, H_Q, H_KV, N, T, v, v_sb, v_sh, v_sn, v_scale, vert_vt8, (cudaStream_t)stream);
}

extern "C" int hq_prefill_quant_v_fp8(const void* v, int64_t v_sb, int64_t v_sh, int64_t v_sn, int B, int H_KV, int N,
                                      void* v_t8, float* v_scale, void* amax_scratch, void* stream) {
  using namespace hq;
  HQ_REQUIRE(v && v_t8 && v_scale && amax_scratch && B > 0 && H_KV > 0 && N > 0, HQ_ERR_INVALID, "hq_prefill_quant_v_fp8: bad arguments");
  HQ_REQUIRE(aligned16(v) && aligned16(v_t8) && v_sb % 8 == 0 && v_sh % 8 == 0 && v_sn % 8 == 0, HQ_ERR_ALIGNMENT,
             "hq_prefill_quant_v_fp8: rows must be 16-byte aligned");
  return prefill_tc_prepare_v_fp8(v, v_sb, v_sh, v_sn, B, H_KV, N, v_t8, v_scale, amax_scratch, (cudaStream_t)stream);
}

extern "C" int hq_prefill_transpose_v(const void* v, int64_t v_sb, int64_t v_sh, int64_t v_sn, int B, int H_KV, int N,
                                      void* v_t, void* stream) {
  using namespace hq;
  HQ_REQUIRE(v && v_t && B > 0 && H_KV > 0 && N > 0, HQ_ERR_INVALID, "hq_prefill_transpose_v: bad arguments");
  HQ_REQUIRE(aligned16(v) && aligned16(v_t) && v_sb % 8 == 0 && v_sh % 8 == 0 && v_sn % 8 == 0, HQ_ERR_ALIGNMENT,
             "hq_prefill_transpose_v: rows must be 16-byte aligned");
  return prefill_tc_prepare_v(v, v_sb, v_sh, v_sn, B, H_KV, N, v_t, (cudaStream_t)stream);
}

extern "C" int hq_prefill_vertical_prepare(const int32_t* vidx_asc, int B, int H_Q, int H_KV, int N, int window, int T,
                                           const void* k_bf, const void* v, int64_t v_sb, int64_t v_sh, int64_t v_sn,
                                           const float* k_scale, void* vert_k, void* vert_vt, float* k_bias,
                                           int32_t* nv_valid, void* stream) {
  using namespace hq;
  HQ_REQUIRE(B > 0 && H_Q > 0 && H_KV > 0 && N > 0 && T >= 0 && window >= 0 && H_Q % H_KV == 0, HQ_ERR_INVALID,
             "hq_prefill_vertical_prepare: bad sizes");
  HQ_REQUIRE(k_scale && k_bias, HQ_ERR_INVALID, "hq_prefill_vertical_prepare: k_scale / k_bias missing");
  HQ_REQUIRE(T == 0 || (vidx_asc && k_bf && v && vert_k && vert_vt && nv_valid), HQ_ERR_INVALID,
             "hq_prefill_vertical_prepare: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const int nqb = (N + 127) / 128, Npad = (N + 63) / 64 * 64;
  // (b, hq) -> (b, hq / R) as one division of the flat index needs R to divide H_Q, checked above
  vertical_meta_kernel<<<B * H_Q, 256, 0, st>>>(vidx_asc, T, N, Npad, window, nqb, H_Q / H_KV, k_scale, k_bias, nv_valid);
  HQ_CUDA(cudaGetLastError());
  if (T == 0) return HQ_OK;
  HQ_REQUIRE(aligned16(v) && aligned16(k_bf) && aligned16(vert_k) && aligned16(vert_vt) && v_sb % 8 == 0 &&
                 v_sh % 8 == 0 && v_sn % 8 == 0, HQ_ERR_ALIGNMENT, "hq_prefill_vertical_prepare: rows must be 16-byte aligned");
  return prefill_tc_prepare_vertical(vidx_asc, B, H_Q, H_KV, N, T, k_bf, v, v_sb, v_sh, v_sn, vert_k, vert_vt, st);
}

extern "C" int hq_prefill_hybrid(const hq_prefill_args* a, void* stream) {
  using namespace hq;
  HQ_REQUIRE(a != nullptr, HQ_ERR_INVALID, "hq_prefill_hybrid: null args");
  HQ_REQUIRE(a->struct_bytes == (int32_t)sizeof(hq_prefill_args), HQ_ERR_INVALID, "hq_prefill_hybrid: struct_bytes %d != %d",
             a->struct_bytes, (int)sizeof(hq_prefill_args));
  HQ_REQUIRE(a->head_dim == 128, HQ_ERR_UNSUPPORTED, "hq_prefill_hybrid: head_dim %d (only 128 is built)", a->head_dim);
  HQ_REQUIRE(a->B > 0 && a->H_Q > 0 && a->H_KV > 0 && a->N > 0 && a->H_Q % a->H_KV == 0 && a->window >= 0 && a->T >= 0,
             HQ_ERR_INVALID, "hq_prefill_hybrid: bad sizes");
  HQ_REQUIRE(a->q_i8 && a->q_bf && a->q_scale && a->k_i8 && a->k_bf && a->k_scale && a->k_bias && a->out && a->status,
             HQ_ERR_INVALID, "hq_prefill_hybrid: null pointer");
  if (a->pv_fp8) {
    HQ_REQUIRE(a->v_t8 && a->v_scale8 && aligned16(a->v_t8), HQ_ERR_INVALID, "hq_prefill_hybrid: FP8 P V needs v_t8 (16-byte aligned) and v_scale8");
    HQ_REQUIRE(a->T == 0 || (a->vert_vt8 && aligned16(a->vert_vt8)), HQ_ERR_INVALID, "hq_prefill_hybrid: FP8 P V with vertical lines needs vert_vt8");
  } else {
    HQ_REQUIRE(a->v_t != nullptr, HQ_ERR_INVALID, "hq_prefill_hybrid: v_t is null");
  }
  HQ_REQUIRE(a->T == 0 || (a->vert_k && (a->vert_vt || a->pv_fp8) && a->nv_valid), HQ_ERR_INVALID,
             "hq_prefill_hybrid: vertical arguments missing");
  HQ_REQUIRE(aligned16(a->q_i8) && aligned16(a->q_bf) && aligned16(a->k_i8) && aligned16(a->k_bf) && (a->pv_fp8 || aligned16(a->v_t)) &&
                 aligned16(a->k_scale) && aligned16(a->k_bias) && aligned16(a->out) && a->o_sn % 8 == 0 && a->o_sh % 8 == 0 && a->o_sb % 8 == 0,
             HQ_ERR_ALIGNMENT, "hq_prefill_hybrid: operand rows must be 16-byte aligned");
  HQ_REQUIRE(a->out_dtype == HQ_BF16 || a->out_dtype == HQ_F16 || a->out_dtype == HQ_F32, HQ_ERR_UNSUPPORTED,
             "hq_prefill_hybrid: out_dtype %d", a->out_dtype);
  return prefill_tc_launch(a, (cudaStream_t)stream);
}
