// gtb_seq_latent.cuh -- mechanisms of the pre-norm layer style of the layer-list sequence models:
//   * hyper-connections: the residual stream kept in several copies, read through a weighted sum and rewritten all at once by
//     every sublayer; fused with the norm that feeds the next sublayer (Dynamic Tanh or RMS with a weight vector)
//   * latent attention: keys and values are up-projections of one low-rank latent per token plus one rotary key part shared by the
//     heads; the slot caches only [latent | rotated key part].  Rows are served in the absorbed form: the query's plain part is
//     carried through the key up-projection (q' = uk_h^T q_h), scores and the weighted sum run over the cached latents like a
//     one-K/V-head attention of head size kv_rank + rope_dim (the softmax kernels of gtb_seq_mixers.cuh), and the value
//     up-projection follows on the summed latent.  Prompt portions in bf16 mode expand keys and values of the visible range instead.
//   * gated routed experts: sigmoid router, renormalised top-k weights, SiLU-gated experts, a gated shared expert
//   * soft-capped logits
// Precision follows gtb_seq_kernels.cuh: fp32 everywhere except operands of matrix products and the cache (type OT).
#pragma once
#include "gtb_seq_mixers.cuh"

namespace gtb {
namespace seq {

constexpr int HC_MAX = 8;                   // most copies of the residual stream

// what a sublayer's input norm needs
struct NormArgs {
    int kind;                 // GTB_NORM_RMS: v / sqrt(mean(v^2) + eps) * w;  GTB_NORM_DYT: tanh(alpha v) * w + b
    const float *w, *b, *alpha;
    float eps;
};
__device__ __forceinline__ float silu_(float z) { return z * sigmoidf_(z); }

// One kernel per sublayer boundary.  XS [ns][R][width] are the copies of the stream (src_ns of them valid on entry: 1 right after
// the embedding, which is broadcast).  With hc_prev = [in | out | mix] of the sublayer that has just produced Y (+ Y2):
//     x_t <- sum_s mix[s][t] x_s + out[t] * (Y + Y2)            for all t at once, from the old copies
// (grouped experts: Y = null and the row's share is the sum of rows pair_dst[r * top + k] of Yg, in order of k)
// then, with in_next: u = sum_s in_next[s] x_s of the NEW copies, norm(u) -> the next product's operand; xsum (optional) receives the
// sum of the new copies (what follows the last layer, and what a capture keeps).  One CTA per row.
template <int V> struct HcVec { float v[V]; };
template <int V> __device__ __forceinline__ HcVec<V> hc_load(const float* p) {
    HcVec<V> o;
    if (V == 4) { const float4 t = *reinterpret_cast<const float4*>(p); o.v[0] = t.x; o.v[1] = t.y; o.v[2] = t.z; o.v[3] = t.w; }
    else o.v[0] = *p;
    return o;
}
template <int V> __device__ __forceinline__ void hc_store(float* p, const HcVec<V>& a) {
    if (V == 4) *reinterpret_cast<float4*>(p) = make_float4(a.v[0], a.v[1], a.v[2], a.v[3]);
    else *p = a.v[0];
}
// V = 4: width, ld_op and every base are multiples of four elements (16-byte accesses); V = 1 otherwise.  NSM: the most copies this
// instance takes (its register arrays are that long).  grid (rows, column groups); an RMS norm needs the whole row in one CTA
// (gridDim.y = 1).
template <typename OT, int V, int NSM>
__global__ void __launch_bounds__(256, NSM <= 4 ? 3 : 2) k_hc_step(float* __restrict__ XS, size_t stream_stride, int ns, int src_ns, int width,
                                                 const float* __restrict__ Y, const float* __restrict__ Y2, const float* __restrict__ Yg,
                                                 const int* __restrict__ pair_dst, int top, const float* __restrict__ hc_prev,
                                                 const float* __restrict__ in_next, NormArgs nrm, OT* __restrict__ op, int ld_op,
                                                 float* __restrict__ xsum) {
    __shared__ float red[33];
    __shared__ float sh[2 * HC_MAX + HC_MAX * HC_MAX + HC_MAX];
    __shared__ int sdst[PN_MAX_TOP];
    const int r = blockIdx.x;
    if (Yg && threadIdx.x < top) sdst[threadIdx.x] = pair_dst[(size_t)r * top + threadIdx.x];
    float* s_out = sh + HC_MAX;               // (sh: in of the previous sublayer, unused) | out | mix | in_next
    float* s_mix = sh + 2 * HC_MAX;
    float* s_in = sh + 2 * HC_MAX + HC_MAX * HC_MAX;
    if (threadIdx.x < ns) {
        if (hc_prev) {
            s_out[threadIdx.x] = hc_prev[ns + threadIdx.x];
            for (int t = 0; t < ns; t++) s_mix[threadIdx.x * ns + t] = hc_prev[2 * ns + threadIdx.x * ns + t];
        }
        if (in_next) s_in[threadIdx.x] = in_next[threadIdx.x];
    }
    __syncthreads();
    const bool rms = in_next && nrm.kind == 0;
    const float alpha = (in_next && !rms) ? nrm.alpha[0] : 0.0f;
    float ss = 0.0f;
    // pass 1 rewrites the copies (and gathers the mean square of u for an RMS norm); pass 2 (RMS only) re-reads them
    for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * V; c < width; c += gridDim.y * blockDim.x * V) {
        const size_t at = (size_t)r * width + c;
        HcVec<V> xo[NSM], y, u, sum;
#pragma unroll
        for (int s = 0; s < NSM; s++)
            if (s < ns) xo[s] = hc_load<V>(XS + (size_t)(s < src_ns ? s : 0) * stream_stride + at);
#pragma unroll
        for (int i = 0; i < V; i++) y.v[i] = u.v[i] = sum.v[i] = 0.0f;
        if (hc_prev) {
            if (Yg) {
                for (int k = 0; k < top; k++) {
                    const HcVec<V> g = hc_load<V>(Yg + (size_t)sdst[k] * width + c);
#pragma unroll
                    for (int i = 0; i < V; i++) y.v[i] += g.v[i];
                }
            } else y = hc_load<V>(Y + at);
            if (Y2) {
                const HcVec<V> g = hc_load<V>(Y2 + at);
#pragma unroll
                for (int i = 0; i < V; i++) y.v[i] += g.v[i];
            }
        }
#pragma unroll
        for (int t = 0; t < NSM; t++)
            if (t < ns) {
                HcVec<V> xt = xo[t];
                if (hc_prev) {
#pragma unroll
                    for (int i = 0; i < V; i++) {
                        float a = s_out[t] * y.v[i];
#pragma unroll
                        for (int s = 0; s < NSM; s++)
                            if (s < ns) a = fmaf(s_mix[s * ns + t], xo[s].v[i], a);
                        xt.v[i] = a;
                    }
                }
                if (hc_prev || t >= src_ns) hc_store<V>(XS + (size_t)t * stream_stride + at, xt);
#pragma unroll
                for (int i = 0; i < V; i++) {
                    sum.v[i] += xt.v[i];
                    if (in_next) u.v[i] = fmaf(s_in[t], xt.v[i], u.v[i]);
                }
            }
        if (xsum) hc_store<V>(xsum + at, sum);
        if (in_next) {
            if (rms) {
#pragma unroll
                for (int i = 0; i < V; i++) ss += u.v[i] * u.v[i];
            } else {
                float o[V];
#pragma unroll
                for (int i = 0; i < V; i++) o[i] = fmaf(tanhf(alpha * u.v[i]), nrm.w[c + i], nrm.b[c + i]);
                if (V == 4) store4(op + (size_t)r * ld_op + c, o[0], o[1], o[2], o[3]);
                else op[(size_t)r * ld_op + c] = cvt<OT>(o[0]);
            }
        }
    }
    if (!rms) return;
    ss = block_sum(ss, red);
    const float sc = 1.0f / sqrtf(ss / (float)width + nrm.eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float u = 0.0f;
        for (int t = 0; t < ns; t++) u = fmaf(s_in[t], XS[(size_t)t * stream_stride + (size_t)r * width + c], u);
        op[(size_t)r * ld_op + c] = cvt<OT>(u * sc * nrm.w[c]);
    }
}

// out = tanh(alpha x) * w + b of gathered rows (the model's output norm)
template <typename OUT>
__global__ void __launch_bounds__(256) k_dyt_rows(const float* __restrict__ x, int width, NormArgs nrm, const int* __restrict__ rows,
                                                  OUT* __restrict__ out, int ld_out) {
    const int o = blockIdx.x, r = rows ? rows[o] : o;
    const float a = nrm.alpha[0];
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        out[(size_t)o * ld_out + c] = cvt<OUT>(fmaf(tanhf(a * x[(size_t)r * width + c]), nrm.w[c], nrm.b[c]));
}

__global__ void k_softcap(float* __restrict__ v, size_t n, float cap) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) v[i] = cap * tanhf(v[i] / cap);
}

// ------------------------------------------------------------------------------------------------ latent attention
struct LatAttn {
    int heads, dim, rope, vdim, rank, q_rank;     // dim: plain query/key entries per head; rope: rotated ones
    int rot_dims, rot_layout;
    const float* inv_freq;       // [rot_dims / 2]
    const float *kv_norm, *q_norm;
    float eps;
    int q_off, kv_off, g_off;    // columns of [q | dq], dkv and the gates in the projection buffer
    int a_off;
    int c_ld;                    // row stride of the latent cache [n_slots][max_ctx][c_ld]: latent, then the rotated key part
    int max_ctx;
};
__device__ __forceinline__ void rot_pair(const LatAttn& b, int pr, int& i0, int& i1) {
    i0 = b.rot_layout ? 2 * pr : pr;
    i1 = b.rot_layout ? 2 * pr + 1 : pr + b.rot_dims / 2;
}

// per row: latent = unit-RMS(dkv[:rank]) * kv_norm and the rotated key part -> the slot's cache row (CTA y = 0); with a query latent,
// unit-RMS(dq) * q_norm -> the operand of the query up-projection, zero-padded to ld_q (CTA y = 1)
template <typename OT>
__global__ void __launch_bounds__(128) k_lat_prep(PassTables t, LatAttn b, const float* __restrict__ P, int ldp, OT* __restrict__ cache,
                                                  OT* __restrict__ opq, int ld_q) {
    __shared__ float red[33];
    const int r = blockIdx.x;
    const int slot = t.seg_slot[t.row_seg[r]], pos = t.row_pos[r];
    const float* p = P + (size_t)r * ldp;
    if (blockIdx.y == 1) {                               // the query latent (grid y = 2 only with one)
        float sq_ = 0.0f;
        for (int i = threadIdx.x; i < b.q_rank; i += blockDim.x) { const float v = p[b.q_off + i]; sq_ += v * v; }
        sq_ = block_sum(sq_, red);
        const float sc = 1.0f / sqrtf(sq_ / (float)b.q_rank + b.eps);
        for (int i = threadIdx.x; i < ld_q; i += blockDim.x) opq[(size_t)r * ld_q + i] = cvt<OT>(i < b.q_rank ? p[b.q_off + i] * sc * b.q_norm[i] : 0.0f);
        return;
    }
    OT* dst = cache + ((size_t)slot * b.max_ctx + pos) * b.c_ld;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < b.rank; i += blockDim.x) { const float v = p[b.kv_off + i]; ss += v * v; }
    ss = block_sum(ss, red);
    float sc = 1.0f / sqrtf(ss / (float)b.rank + b.eps);
    for (int i = threadIdx.x; i < b.rank; i += blockDim.x) dst[i] = cvt<OT>(p[b.kv_off + i] * sc * b.kv_norm[i]);
    const float* kr = p + b.kv_off + b.rank;
    const float fpos = (float)pos;
    for (int pr = threadIdx.x; pr < b.rot_dims / 2; pr += blockDim.x) {
        int i0, i1;
        rot_pair(b, pr, i0, i1);
        float sn, cs;
        sincosf(fpos * b.inv_freq[pr], &sn, &cs);
        dst[b.rank + i0] = cvt<OT>(kr[i0] * cs - kr[i1] * sn);
        dst[b.rank + i1] = cvt<OT>(kr[i1] * cs + kr[i0] * sn);
    }
    for (int i = b.rot_dims + threadIdx.x; i < b.rope; i += blockDim.x) dst[b.rank + i] = cvt<OT>(kr[i]);
}

// Prompt portions: the heads' queries with their rotated part turned to the row's position, and the heads' gate logits behind them:
// QR [R][ld_qr] = [heads x (plain | rotated) | heads gates].  Q may be QR itself (in place).
__global__ void __launch_bounds__(128) k_lat_qrot(PassTables t, LatAttn b, const float* __restrict__ Q, int ldq, int q0, const float* __restrict__ P, int ldp,
                                                  float* __restrict__ QR, int ld_qr) {
    const int r = blockIdx.x, hd = b.dim + b.rope;
    const float fpos = (float)t.row_pos[r];
    const float* q = Q + (size_t)r * ldq + q0;
    float* o = QR + (size_t)r * ld_qr;
    const int half = b.rot_dims / 2;
    for (int e = threadIdx.x; e < b.heads * hd; e += blockDim.x) {
        const int h = e / hd, i = e % hd, j = i - b.dim;
        if (j < 0 || j >= b.rot_dims) { if (o + e != q + e) o[e] = q[e]; continue; }
        const int pr = b.rot_layout ? j >> 1 : (j < half ? j : j - half);
        const bool first = b.rot_layout ? (j & 1) == 0 : j < half;
        if (!first) continue;                     // the pair's first entry writes both
        int i0, i1;
        rot_pair(b, pr, i0, i1);
        float sn, cs;
        sincosf(fpos * b.inv_freq[pr], &sn, &cs);
        const float u = q[h * hd + b.dim + i0], v = q[h * hd + b.dim + i1];
        o[h * hd + b.dim + i0] = u * cs - v * sn;
        o[h * hd + b.dim + i1] = v * cs + u * sn;
    }
    if (P) for (int h = threadIdx.x; h < b.heads; h += blockDim.x) o[b.heads * hd + h] = P[(size_t)r * ldp + b.g_off + h];
}

// Expanded keys and values of n cached tokens of one slot from position lo: X [n][heads * (dim + vdim)] (fp32) holds [uk c | uv c];
// Kx [n_slots][max_ctx][heads][dim + rope] <- [plain key | the cached rotated part], Vx [n_slots][max_ctx][heads][vdim].
__global__ void __launch_bounds__(256) k_lat_pack(LatAttn b, const float* __restrict__ X, int n, int slot, int lo, const bf16* __restrict__ cache,
                                                  bf16* __restrict__ Kx, bf16* __restrict__ Vx) {
    const int j = blockIdx.x, hd = b.dim + b.rope;
    const size_t row = (size_t)slot * b.max_ctx + lo + j;
    const float* x = X + (size_t)j * b.heads * (b.dim + b.vdim);
    const bf16* cr = cache + row * b.c_ld + b.rank;
    bf16* k = Kx + row * (size_t)(b.heads * hd);
    bf16* v = Vx + row * (size_t)(b.heads * b.vdim);
    for (int e = threadIdx.x; e < b.heads * hd; e += blockDim.x) {
        const int h = e / hd, i = e % hd;
        k[e] = i < b.dim ? __float2bfloat16_rn(x[h * b.dim + i]) : cr[i - b.dim];
    }
    const float* xv = x + b.heads * b.dim;
    for (int e = threadIdx.x; e < b.heads * b.vdim; e += blockDim.x) v[e] = __float2bfloat16_rn(xv[e]);
}

// Absorbed query of (row, head): qa[0 .. rank) = sum_d q_plain[d] uk[head * dim + d][:], qa[rank ..) = the rotated part at the row's
// position.  Q [R][ldq] holds the heads' [plain | rotated] queries from column q0; QA [R][heads * (rank + rope)].  uk [heads * dim][ld_uk],
// ld_uk a multiple of 64 with zero columns beyond rank.  grid (rows, heads, groups of 128 latent columns); the CTA's four warps split
// the plain entries, a lane takes four adjacent columns (one 8-byte load per entry), the warps' sums meet in shared memory.
__global__ void __launch_bounds__(128) k_lat_qabs(PassTables t, LatAttn b, const float* __restrict__ Q, int ldq, int q0, const bf16* __restrict__ uk, int ld_uk,
                                                  float* __restrict__ QA) {
    extern __shared__ float sq[];             // [dim + rope], then [4][128] partial sums
    const int r = blockIdx.x, h = blockIdx.y, hd = b.dim + b.rope;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* part = sq + hd;
    const float* q = Q + (size_t)r * ldq + q0 + (size_t)h * hd;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) sq[i] = q[i];
    __syncthreads();
    float* qa = QA + ((size_t)r * b.heads + h) * (b.rank + b.rope);
    const int c = blockIdx.z * 128 + lane * 4;
    float a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (c < b.rank) {
        const bf16* w = uk + (size_t)h * b.dim * ld_uk + c;
        const int d0 = (b.dim * warp) / 4, d1 = (b.dim * (warp + 1)) / 4;
#pragma unroll 8
        for (int d = d0; d < d1; d++) {
            const uint2 wv = __ldg(reinterpret_cast<const uint2*>(w + (size_t)d * ld_uk));
            const float qd = sq[d];
            a[0] = fmaf(qd, __uint_as_float(wv.x << 16), a[0]);
            a[1] = fmaf(qd, __uint_as_float(wv.x & 0xffff0000u), a[1]);
            a[2] = fmaf(qd, __uint_as_float(wv.y << 16), a[2]);
            a[3] = fmaf(qd, __uint_as_float(wv.y & 0xffff0000u), a[3]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) part[warp * 128 + lane * 4 + i] = a[i];
    __syncthreads();
    {
        const int cc = blockIdx.z * 128 + threadIdx.x;
        if (cc < b.rank) qa[cc] = (part[threadIdx.x] + part[128 + threadIdx.x]) + (part[256 + threadIdx.x] + part[384 + threadIdx.x]);
    }
    if (blockIdx.z != 0) return;
    const float fpos = (float)t.row_pos[r];
    const float* qr = sq + b.dim;
    for (int pr = threadIdx.x; pr < b.rot_dims / 2; pr += blockDim.x) {
        int i0, i1;
        rot_pair(b, pr, i0, i1);
        float sn, cs;
        sincosf(fpos * b.inv_freq[pr], &sn, &cs);
        qa[b.rank + i0] = qr[i0] * cs - qr[i1] * sn;
        qa[b.rank + i1] = qr[i1] * cs + qr[i0] * sn;
    }
    for (int i = b.rot_dims + threadIdx.x; i < b.rope; i += blockDim.x) qa[b.rank + i] = qr[i];
}

// Decode rows in bf16 mode: the absorbed form on tensor cores.  All heads of a row share the cached latents, so a CTA takes 16 heads as
// the M dimension of mma.sync m16n8k16 and sweeps its share of the row's keys (grid: rows x groups of 16 heads x key splits) in tiles
// of 64: the tile [64][latent | rotated part] is staged once in shared memory as bf16 and serves both products -- S = Q' K^T (each of
// the four warps scores 16 keys), softmax weights in fp32 against the running maximum (the warps' row maxima meet in shared memory),
// O += P V with V = the tile's latent columns (each warp owns VPW value columns, P comes back from shared memory as bf16 A fragments).
// Leaves (maximum, denominator, unnormalised sum) per head in part [split][R][heads][rank + 2], which k_sattn_join folds with the sink.
// b: the one-K/V-head view of the branch (dim = rank + rope, vdim = rank, k_ld = the cache's row stride).
template <int VPW>
__global__ void __launch_bounds__(128) k_lat_dec_mma(PassTables t, SoftAttn b, const float* __restrict__ QA, int ldqa, const bf16* __restrict__ cache,
                                                     float* __restrict__ part, int R) {
    constexpr int TK = 64;
    extern __shared__ __align__(16) unsigned char ld_raw[];
    const int D = b.dim, DP = (D + 15) & ~15, LK = DP + 8, LP = TK + 8;
    bf16* sq = reinterpret_cast<bf16*>(ld_raw);          // [16][LK]
    bf16* sk = sq + 16 * LK;                             // [TK][LK]
    bf16* sp = sk + TK * LK;                             // [16][LP]
    float* smx = reinterpret_cast<float*>(sp + 16 * LP); // [4][16] row maxima of the warps' key groups, then their row sums
    const int r = blockIdx.x, h0 = blockIdx.y * 16, pos = t.row_pos[r], slot = t.seg_slot[t.row_seg[r]];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
    const int lo = b.window > 0 ? max(0, pos - b.window + 1) : 0, total = pos - lo + 1;
    const int per = ((total + (int)gridDim.z - 1) / (int)gridDim.z + TK - 1) / TK * TK;
    const int n_lo = blockIdx.z * per, n_hi = min(total, n_lo + per);
    const int nh = min(16, b.heads - h0);
    float* out = part + (((size_t)blockIdx.z * R + r) * b.heads + h0) * (b.vdim + 2);
    if (n_lo >= n_hi) {
        if (threadIdx.x < nh) { out[(size_t)threadIdx.x * (b.vdim + 2)] = -INFINITY; out[(size_t)threadIdx.x * (b.vdim + 2) + 1] = 0.0f; }
        return;
    }
    const bf16* kbase = cache + ((size_t)slot * b.max_ctx + lo) * b.k_ld;
    const bool vec = (D % 8 == 0) && (b.k_ld % 8 == 0);
    const uint32_t sq_a = (uint32_t)__cvta_generic_to_shared(sq), sk_a = (uint32_t)__cvta_generic_to_shared(sk), sp_a = (uint32_t)__cvta_generic_to_shared(sp);
    // keys j0 .. of the range -> the tile in shared memory (asynchronous 16-byte copies when the cache rows allow them)
    auto load_tile = [&](int j0) {
        const int nk = min(TK, n_hi - j0);
        if (vec) {
            for (int e = threadIdx.x; e < TK * (DP / 8); e += 128) {
                const int rr = e / (DP / 8), c8 = (e % (DP / 8)) * 8;
                const bool ok = rr < nk && c8 < D;
                sa_cp16(sk_a + (uint32_t)((rr * LK + c8) * 2), ok ? (const void*)(kbase + (size_t)(j0 + rr) * b.k_ld + c8) : (const void*)kbase, ok);
            }
        } else {
            for (int e = threadIdx.x; e < TK * DP; e += 128) {
                const int rr = e / DP, i = e % DP;
                sk[rr * LK + i] = (rr < nk && i < D) ? kbase[(size_t)(j0 + rr) * b.k_ld + i] : __float2bfloat16_rn(0.0f);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    load_tile(n_lo);                                     // in flight while the queries are staged
    const float* qsrc = QA + (size_t)r * ldqa + (size_t)h0 * D;      // the group's heads are contiguous: nh x D floats
    if (D % 4 == 0 && ldqa % 4 == 0) {
        for (int e = threadIdx.x; e < 16 * (DP - D) + (16 - nh) * D; e += 128) {      // zero the padding: columns D .. DP of every row, rows nh .. 16
            const int npc = 16 * (DP - D);
            if (e < npc) sq[(e / (DP - D)) * LK + D + e % (DP - D)] = __float2bfloat16_rn(0.0f);
            else sq[(nh + (e - npc) / D) * LK + (e - npc) % D] = __float2bfloat16_rn(0.0f);
        }
#pragma unroll 4
        for (int e = threadIdx.x * 4; e < nh * D; e += 512) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(qsrc + e));
            bf16* dst = sq + (e / D) * LK + e % D;
            *reinterpret_cast<uint32_t*>(dst) = sa_pack(v.x, v.y);
            *reinterpret_cast<uint32_t*>(dst + 2) = sa_pack(v.z, v.w);
        }
    } else {
        for (int e = threadIdx.x; e < 16 * DP; e += 128) {
            const int hh = e / DP, i = e % DP;
            sq[hh * LK + i] = __float2bfloat16_rn((hh < nh && i < D) ? qsrc[(size_t)hh * D + i] : 0.0f);
        }
    }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;
    float o[VPW / 8][4];
#pragma unroll
    for (int n = 0; n < VPW / 8; n++) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f; }
    for (int j0 = n_lo; j0 < n_hi; j0 += TK) {
        const int nk = min(TK, n_hi - j0);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        // scores of this warp's 16 keys for the 16 heads
        float sc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
        for (int kk = 0; kk < DP / 16; kk++) {
            uint32_t a[4], b0, b1, b2, b3;
            sa_ldsm_x4(sq_a + (uint32_t)((((lane & 15)) * LK + kk * 16 + (lane >> 4) * 8) * 2), a[0], a[1], a[2], a[3]);
            sa_ldsm_x4(sk_a + (uint32_t)(((warp * 16 + (lane & 7) + (lane >> 4) * 8) * LK + kk * 16 + ((lane >> 3) & 1) * 8) * 2), b0, b1, b2, b3);
            sa_mma(sc[0], a, b0, b1);
            sa_mma(sc[1], a, b2, b3);
        }
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int n = 0; n < 2; n++)
#pragma unroll
            for (int x = 0; x < 4; x++) {
                const bool vis = warp * 16 + n * 8 + tq * 2 + (x & 1) < nk;
                const float sv = vis ? sc[n][x] * b.scale : -INFINITY;
                sc[n][x] = sv;
                if (x >= 2) mx_hi = fmaxf(mx_hi, sv); else mx_lo = fmaxf(mx_lo, sv);
            }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1)); mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1)); mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        if (tq == 0) { smx[warp * 16 + gq] = mx_lo; smx[warp * 16 + gq + 8] = mx_hi; }
        __syncthreads();
        const float mn_lo = fmaxf(m_lo, fmaxf(fmaxf(smx[gq], smx[16 + gq]), fmaxf(smx[32 + gq], smx[48 + gq])));          // the tile's first key is always visible
        const float mn_hi = fmaxf(m_hi, fmaxf(fmaxf(smx[gq + 8], smx[24 + gq]), fmaxf(smx[40 + gq], smx[56 + gq])));
        const float c_lo = m_lo == -INFINITY ? 0.0f : __expf(m_lo - mn_lo), c_hi = m_hi == -INFINITY ? 0.0f : __expf(m_hi - mn_hi);
        m_lo = mn_lo; m_hi = mn_hi;
        l_lo *= c_lo; l_hi *= c_hi;
#pragma unroll
        for (int n = 0; n < VPW / 8; n++) { o[n][0] *= c_lo; o[n][1] *= c_lo; o[n][2] *= c_hi; o[n][3] *= c_hi; }
#pragma unroll
        for (int n = 0; n < 2; n++) {
            const float w0 = sc[n][0] == -INFINITY ? 0.0f : __expf(sc[n][0] - mn_lo), w1 = sc[n][1] == -INFINITY ? 0.0f : __expf(sc[n][1] - mn_lo);
            const float w2 = sc[n][2] == -INFINITY ? 0.0f : __expf(sc[n][2] - mn_hi), w3 = sc[n][3] == -INFINITY ? 0.0f : __expf(sc[n][3] - mn_hi);
            l_lo += w0 + w1; l_hi += w2 + w3;
            const int col = warp * 16 + n * 8 + tq * 2;
            *reinterpret_cast<uint32_t*>(sp + gq * LP + col) = sa_pack(w0, w1);
            *reinterpret_cast<uint32_t*>(sp + (gq + 8) * LP + col) = sa_pack(w2, w3);
        }
        __syncthreads();
        // this warp's VPW value columns over all 64 keys of the tile
        const int cw = warp * VPW;
#pragma unroll
        for (int kk = 0; kk < TK / 16; kk++) {
            uint32_t a[4];
            sa_ldsm_x4(sp_a + (uint32_t)(((lane & 15) * LP + kk * 16 + (lane >> 4) * 8) * 2), a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int n2 = 0; n2 < VPW / 16; n2++) {
                if (cw + n2 * 16 >= DP) continue;                 // beyond the staged columns (ranks that are no multiple of 4 * VPW)
                uint32_t b0, b1, b2, b3;
                sa_ldsm_x4_t(sk_a + (uint32_t)(((kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LK + cw + n2 * 16 + (lane >> 4) * 8) * 2), b0, b1, b2, b3);
                sa_mma(o[2 * n2], a, b0, b1);
                sa_mma(o[2 * n2 + 1], a, b2, b3);
            }
        }
        __syncthreads();                                         // the tile and the weights may be overwritten
        if (j0 + TK < n_hi) load_tile(j0 + TK);
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    if (tq == 0) { smx[warp * 16 + gq] = l_lo; smx[warp * 16 + gq + 8] = l_hi; }
    __syncthreads();
    if (threadIdx.x < nh) {
        const int hh = threadIdx.x;
        out[(size_t)hh * (b.vdim + 2) + 1] = (smx[hh] + smx[16 + hh]) + (smx[32 + hh] + smx[48 + hh]);
    }
    if (warp == 0 && tq == 0) {
        if (gq < nh) out[(size_t)gq * (b.vdim + 2)] = m_lo;
        if (gq + 8 < nh) out[(size_t)(gq + 8) * (b.vdim + 2)] = m_hi;
    }
    const int cw = warp * VPW;
#pragma unroll
    for (int n = 0; n < VPW / 8; n++)
#pragma unroll
        for (int x = 0; x < 2; x++) {
            const int c = cw + n * 8 + tq * 2 + x;
            if (c >= b.vdim) continue;
            if (gq < nh) out[(size_t)gq * (b.vdim + 2) + 2 + c] = o[n][x];
            if (gq + 8 < nh) out[(size_t)(gq + 8) * (b.vdim + 2) + 2 + c] = o[n][2 + x];
        }
}

// Value up-projection of the summed latents and the head's gate: out[r][a_off + h vdim + v] = logistic(P[r][g_off + h]) * uv[h vdim + v] . ol[r][h]
// OL [R][ld_ol] holds heads x rank summed latents; a warp per output entry.  gate 0: no gate.
template <typename OT>
__global__ void __launch_bounds__(256) k_lat_vup(LatAttn b, const OT* __restrict__ OL, int ld_ol, const bf16* __restrict__ uv, int ld_uv,
                                                 const float* __restrict__ P, int ldp, int gate, OT* __restrict__ out, int ld_out) {
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int n = b.heads * b.vdim;
    const bool vec = b.rank % 8 == 0 && ld_ol % 8 == 0 && ld_uv % 8 == 0;
    for (int e = blockIdx.y * nw + warp; e < n; e += gridDim.y * nw) {
        const int h = e / b.vdim;
        const OT* a = OL + (size_t)r * ld_ol + (size_t)h * b.rank;
        const bf16* w = uv + (size_t)e * ld_uv;
        float s = 0.0f;
        if (vec) {
            for (int k = lane * 8; k < b.rank; k += 256) {
                const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w + k));
                float av[8];
                load8<OT>(a + k, av);
                const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    s = fmaf(av[2 * i], __uint_as_float(ww[i] << 16), s);
                    s = fmaf(av[2 * i + 1], __uint_as_float(ww[i] & 0xffff0000u), s);
                }
            }
        } else {
            for (int k = lane; k < b.rank; k += 32) s = fmaf(ldf<OT>(a + k), __bfloat162float(w[k]), s);
        }
        s = warp_sum(s);
        if (lane == 0) {
            if (gate) s *= sigmoidf_(P[(size_t)r * ldp + b.g_off + h]);
            out[(size_t)r * ld_out + b.a_off + e] = cvt<OT>(s);
        }
    }
}

// ------------------------------------------------------------------------------------------------ gated routed experts
// One warp routes one row from its router outputs z [n_exp (+ 1: the shared expert's gate)]: s = logistic(z); the `top` largest s are
// chosen (ties to the lower index) and weighted with s / (sum of the chosen s + 1e-20); shared_w[r] = logistic(z[n_exp]).
// Shared memory: n_exp floats.
__global__ void __launch_bounds__(32) k_moe_route_sigmoid(const float* __restrict__ Z, int ldz, int n_exp, int top, int* __restrict__ sel_idx,
                                                          float* __restrict__ sel_w, float* __restrict__ shared_w) {
    extern __shared__ float ch[];
    const int r = blockIdx.x, lane = threadIdx.x;
    const float* z = Z + (size_t)r * ldz;
    for (int i = lane; i < n_exp; i += 32) ch[i] = sigmoidf_(z[i]);
    __syncwarp();
    float sum = 0.0f;
    for (int k = 0; k < top; k++) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int i = lane; i < n_exp; i += 32) { const float v = ch[i]; if (v > best) { best = v; arg = i; } }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ov > best || (ov == best && oi < arg)) { best = ov; arg = oi; }
        }
        if (arg == 0x7fffffff) { arg = 0; best = 0.0f; }
        sum += best;
        if (lane == 0) { sel_idx[(size_t)r * top + k] = arg; sel_w[(size_t)r * top + k] = best; ch[arg] = -INFINITY; }
        __syncwarp();
    }
    const float inv = 1.0f / (sum + 1e-20f);
    for (int k = lane; k < top; k += 32) sel_w[(size_t)r * top + k] *= inv;
    if (shared_w && lane == 0) shared_w[r] = sigmoidf_(z[n_exp]);
}

// rows of the fused [gate | up] matrix of a gated feed-forward: plain = ff gate rows then ff up rows; interleaved = groups of 32 gate
// rows each followed by their 32 up rows (what the tensor-core epilogue reads)
__device__ __forceinline__ int gu_gate_row(int c, int inter) { return inter ? (c >> 5) * 64 + (c & 31) : c; }
__device__ __forceinline__ int gu_up_row(int c, int ff, int inter) { return inter ? (c >> 5) * 64 + (c & 31) + 32 : ff + c; }

// Few rows: pair (row r, choice k) with expert e streams that expert's gate and up rows once: act[pair][c] = w * silu(gate_e[c] . x_r) *
// (up_e[c] . x_r) for c < ff, zero up to the padded width kfp.  grid (R * top, column groups); a warp takes one column at a time.
// w_gu [n_experts][2 ff][ldw].
template <typename OT>
__global__ void __launch_bounds__(256) k_moe_gu_rows(const OT* __restrict__ X, int ldx, int K, const bf16* __restrict__ w_gu, int ldw, int ff, int kfp,
                                                     int inter, int top, const int* __restrict__ sel_idx, const float* __restrict__ sel_w,
                                                     OT* __restrict__ act) {
    const int pair = blockIdx.x, r = pair / top, e = sel_idx[pair];
    const float wt = sel_w[pair];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const OT* x = X + (size_t)r * ldx;
    const bf16* we = w_gu + (size_t)e * 2 * ff * ldw;
    for (int c = blockIdx.y * nw + warp; c < kfp; c += gridDim.y * nw) {
        float g = 0.0f, u = 0.0f;
        if (c < ff) {
            g = warp_sum(lane_dot<OT>(x, we + (size_t)gu_gate_row(c, inter) * ldw, K, lane));
            u = warp_sum(lane_dot<OT>(x, we + (size_t)gu_up_row(c, ff, inter) * ldw, K, lane));
        }
        if (lane == 0) act[(size_t)pair * kfp + c] = cvt<OT>(wt * silu_(g) * u);
    }
}

// act = row_w[r] * silu(gate) * up from G [R][2 ff] (columns laid out like the rows of the fused matrix) -> operand [R][ld_out], zero-padded
// (grid: rows x column groups; few rows spread their columns over many CTAs)
template <typename OT>
__global__ void k_swiglu_rows(const float* __restrict__ G, int ff, int inter, const float* __restrict__ row_w, OT* __restrict__ out, int ld_out) {
    const int r = blockIdx.x;
    const float wt = row_w ? row_w[r] : 1.0f;
    const float* g = G + (size_t)r * 2 * ff;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < ld_out; c += gridDim.y * blockDim.x)
        out[(size_t)r * ld_out + c] = cvt<OT>(c < ff ? wt * silu_(g[gu_gate_row(c, inter)]) * g[gu_up_row(c, ff, inter)] : 0.0f);
}

}  // namespace seq
}  // namespace gtb
