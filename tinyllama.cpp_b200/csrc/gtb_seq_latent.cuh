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
template <typename OT>
__global__ void __launch_bounds__(256) k_hc_step(float* __restrict__ XS, size_t stream_stride, int ns, int src_ns, int width,
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
    float ss = 0.0f;
    // pass 1 rewrites the copies (and gathers the mean square of u for an RMS norm); pass 2 (RMS only) re-reads them
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float xo[HC_MAX], xn[HC_MAX];
#pragma unroll
        for (int s = 0; s < HC_MAX; s++)
            if (s < ns) xo[s] = XS[(size_t)(s < src_ns ? s : 0) * stream_stride + (size_t)r * width + c];
        if (hc_prev) {
            float y = 0.0f;
            if (Yg) { for (int k = 0; k < top; k++) y += Yg[(size_t)sdst[k] * width + c]; }
            else y = Y[(size_t)r * width + c];
            if (Y2) y += Y2[(size_t)r * width + c];
#pragma unroll
            for (int t = 0; t < HC_MAX; t++)
                if (t < ns) {
                    float a = s_out[t] * y;
#pragma unroll
                    for (int s = 0; s < HC_MAX; s++)
                        if (s < ns) a = fmaf(s_mix[s * ns + t], xo[s], a);
                    xn[t] = a;
                }
        } else {
#pragma unroll
            for (int t = 0; t < HC_MAX; t++) if (t < ns) xn[t] = xo[t];
        }
        float u = 0.0f, sum = 0.0f;
#pragma unroll
        for (int t = 0; t < HC_MAX; t++)
            if (t < ns) {
                if (hc_prev || t >= src_ns) XS[(size_t)t * stream_stride + (size_t)r * width + c] = xn[t];
                sum += xn[t];
                if (in_next) u = fmaf(s_in[t], xn[t], u);
            }
        if (xsum) xsum[(size_t)r * width + c] = sum;
        if (in_next) {
            if (rms) ss += u * u;
            else op[(size_t)r * ld_op + c] = cvt<OT>(fmaf(tanhf(nrm.alpha[0] * u), nrm.w[c], nrm.b[c]));
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

// per row: latent = unit-RMS(dkv[:rank]) * kv_norm and the rotated key part -> the slot's cache row; with a query latent,
// unit-RMS(dq) * q_norm -> the operand of the query up-projection (zero-padded to ld_q)
template <typename OT>
__global__ void __launch_bounds__(128) k_lat_prep(PassTables t, LatAttn b, const float* __restrict__ P, int ldp, OT* __restrict__ cache,
                                                  OT* __restrict__ opq, int ld_q) {
    __shared__ float red[33];
    const int r = blockIdx.x;
    const int slot = t.seg_slot[t.row_seg[r]], pos = t.row_pos[r];
    const float* p = P + (size_t)r * ldp;
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
    if (b.q_rank > 0) {
        ss = 0.0f;
        for (int i = threadIdx.x; i < b.q_rank; i += blockDim.x) { const float v = p[b.q_off + i]; ss += v * v; }
        ss = block_sum(ss, red);
        sc = 1.0f / sqrtf(ss / (float)b.q_rank + b.eps);
        for (int i = threadIdx.x; i < ld_q; i += blockDim.x) opq[(size_t)r * ld_q + i] = cvt<OT>(i < b.q_rank ? p[b.q_off + i] * sc * b.q_norm[i] : 0.0f);
    }
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
// position.  Q [R][ldq] holds the heads' [plain | rotated] queries from column q0; QA [R][heads * (rank + rope)].  uk [heads * dim][ld_uk].
__global__ void __launch_bounds__(128) k_lat_qabs(PassTables t, LatAttn b, const float* __restrict__ Q, int ldq, int q0, const bf16* __restrict__ uk, int ld_uk,
                                                  float* __restrict__ QA) {
    extern __shared__ float sq[];             // [dim + rope]
    const int r = blockIdx.x, h = blockIdx.y, hd = b.dim + b.rope;
    const float* q = Q + (size_t)r * ldq + q0 + (size_t)h * hd;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) sq[i] = q[i];
    __syncthreads();
    float* qa = QA + ((size_t)r * b.heads + h) * (b.rank + b.rope);
    const bf16* w = uk + (size_t)h * b.dim * ld_uk;
    for (int c = threadIdx.x; c < b.rank; c += blockDim.x) {
        float a0 = 0.0f, a1 = 0.0f;
        int d = 0;
        for (; d + 1 < b.dim; d += 2) {
            a0 = fmaf(sq[d], __bfloat162float(w[(size_t)d * ld_uk + c]), a0);
            a1 = fmaf(sq[d + 1], __bfloat162float(w[(size_t)(d + 1) * ld_uk + c]), a1);
        }
        if (d < b.dim) a0 = fmaf(sq[d], __bfloat162float(w[(size_t)d * ld_uk + c]), a0);
        qa[c] = a0 + a1;
    }
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
template <typename OT>
__global__ void k_swiglu_rows(const float* __restrict__ G, int ff, int inter, const float* __restrict__ row_w, OT* __restrict__ out, int ld_out) {
    const int r = blockIdx.x;
    const float wt = row_w ? row_w[r] : 1.0f;
    const float* g = G + (size_t)r * 2 * ff;
    for (int c = threadIdx.x; c < ld_out; c += blockDim.x)
        out[(size_t)r * ld_out + c] = cvt<OT>(c < ff ? wt * silu_(g[gu_gate_row(c, inter)]) * g[gu_up_row(c, ff, inter)] : 0.0f);
}

}  // namespace seq
}  // namespace gtb
