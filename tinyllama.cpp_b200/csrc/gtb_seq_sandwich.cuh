// gtb_seq_sandwich.cuh -- mechanisms of the sandwich layer style of the layer-list sequence models (a norm in front of and behind each
// sublayer):
//   * layer norm / RMS norm with a weight (and bias) as an operand producer, and the residual update x += norm_b(sublayer output) that
//     also writes the NEXT sublayer's normalised input
//   * one RMS norm over a whole query / key projection (its scale per row), for softmax attention with qk_norm 3
//   * differential attention: the combination of a head's two score maps, its unit-RMS norm and gate
//   * retention with SiLU-activated inputs, an RMS norm over the concatenated heads and a logistic gate
//   * a sigmoid router whose choice is limited to the best groups of experts
// The attention and retention kernels themselves are those of gtb_seq_mixers*.cuh and gtb_seq_kernels.cuh.
//
// Precision follows gtb_seq_kernels.cuh: everything below is fp32 except operands of matrix products (type OT).
#pragma once
#include "gtb_seq_latent.cuh"

namespace gtb {
namespace seq {

constexpr int SW_NORM_LAYER = 2;            // NormArgs::kind of a layer norm (GTB_NORM_LAYER); anything else here: RMS with a plain weight

// Sum over the block with ONE barrier: every warp leaves its partial sum in `slot` (32 floats that no other reduction of the kernel uses, so
// nothing has to wait for earlier readers) and every thread adds the partial sums itself, in the same order.
__device__ __forceinline__ float sw_block_sum(float v, float* slot) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) slot[wid] = v;
    __syncthreads();
    float t = 0.0f;
    for (int w = 0; w < nw; w++) t += slot[w];
    return t;
}
// mean and 1 / sqrt(variance + eps) of a row (layer norm), or 0 and 1 / sqrt(mean square + eps) (RMS); a thread holds the values of columns
// (threadIdx.x + i blockDim.x) * 4 .. + 3 in v[4 i ..].  The mean first, then the squared deviations: no cancellation between two large sums.
// red: 64 floats of shared memory of this call's own.
template <int N4>
__device__ __forceinline__ void sw_stats(const float (&v)[4 * N4], int width, int center, float eps, float* red, float& mean, float& rstd) {
    mean = 0.0f;
    if (center) {
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < N4; i++)
            if ((int)(threadIdx.x + i * blockDim.x) * 4 < width) s += (v[4 * i] + v[4 * i + 1]) + (v[4 * i + 2] + v[4 * i + 3]);
        mean = sw_block_sum(s, red) / (float)width;
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < N4; i++)
        if ((int)(threadIdx.x + i * blockDim.x) * 4 < width) {
            const float d0 = v[4 * i] - mean, d1 = v[4 * i + 1] - mean, d2 = v[4 * i + 2] - mean, d3 = v[4 * i + 3] - mean;
            ss += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
        }
    rstd = 1.0f / sqrtf(sw_block_sum(ss, red + 32) / (float)width + eps);
}

// out = norm(x[rows[o]]) as a product operand.  rows: optional gather.
template <typename OT>
__global__ void __launch_bounds__(256) k_norm_rows(const float* __restrict__ x, int width, NormArgs nrm, const int* __restrict__ rows, OT* __restrict__ out, int ld_out) {
    __shared__ float red[33];
    const int o = blockIdx.x, r = rows ? rows[o] : o, center = nrm.kind == SW_NORM_LAYER;
    const float* xr = x + (size_t)r * width;
    float mean = 0.0f;
    if (center) {
        float s = 0.0f;
        for (int c = threadIdx.x; c < width; c += blockDim.x) s += xr[c];
        mean = block_sum(s, red) / (float)width;
    }
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) { const float d = xr[c] - mean; ss += d * d; }
    const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)width + nrm.eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        out[(size_t)o * ld_out + c] = cvt<OT>((xr[c] - mean) * rstd * nrm.w[c] + (center ? nrm.b[c] : 0.0f));
}

// ------------------------------------------------------------------------------------------------ group-limited sigmoid router
// One warp routes one row from its router outputs z [n_exp]: s = logistic(z).  The experts form n_groups equal groups of neighbours; a
// group ranks by the sum of its two largest s (its only s when it has one expert); experts outside the `keep` best groups (ties to the
// lower group) cannot be chosen.  The `top` largest s among the rest are chosen (ties to the lower index) with weight scale * s.  Choices
// top .. top + n_always - 1 are the experts n_exp .. n_exp + n_always - 1 with weight 1 (parts of an expert that every row uses).
// sel_idx / sel_w: the row's top + n_always entries.  s, ch: n_exp floats of shared memory each; gr: n_groups floats.
__device__ __forceinline__ void route_grouped_row(const float* __restrict__ z, int n_exp, int n_groups, int keep, int top, float scale, int n_always,
                                                  int* __restrict__ sel_idx, float* __restrict__ sel_w, float* s, float* ch, float* gr, int lane) {
    for (int i = lane; i < n_exp; i += 32) { const float v = sigmoidf_(z[i]); s[i] = v; ch[i] = v; }
    __syncwarp();
    if (n_groups > 1 && keep < n_groups) {
        const int size = n_exp / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float m1 = -INFINITY, m2 = -INFINITY;
            for (int i = 0; i < size; i++) { const float v = s[g * size + i]; if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) m2 = v; }
            gr[g] = size > 1 ? m1 + m2 : m1;
        }
        __syncwarp();
        // `keep` rounds of arg-max over the groups; a kept group's rank becomes +inf, and what is finite afterwards is closed
        for (int k = 0; k < keep; k++) {
            float best = -INFINITY;
            int arg = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32) { const float v = gr[g]; if (v != INFINITY && v > best) { best = v; arg = g; } }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
                if (ov > best || (ov == best && oi < arg)) { best = ov; arg = oi; }
            }
            if (arg != 0x7fffffff && lane == 0) gr[arg] = INFINITY;
            __syncwarp();
        }
        for (int i = lane; i < n_exp; i += 32) if (gr[i / size] != INFINITY) ch[i] = -INFINITY;
        __syncwarp();
    }
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
        if (lane == 0) { sel_idx[k] = arg; sel_w[k] = best * scale; ch[arg] = -INFINITY; }
        __syncwarp();
    }
    for (int k = lane; k < n_always; k += 32) { sel_idx[top + k] = n_exp + k; sel_w[top + k] = 1.0f; }
}
// rows of router logits Z -> choices; sel_idx / sel_w [rows][top + n_always].  Shared memory: 2 n_exp + n_groups floats.
__global__ void __launch_bounds__(32) k_moe_route_grouped(const float* __restrict__ Z, int ldz, int n_exp, int n_groups, int keep, int top, float scale,
                                                          int n_always, int* __restrict__ sel_idx, float* __restrict__ sel_w) {
    extern __shared__ float rsm[];
    const int r = blockIdx.x, tt = top + n_always;
    route_grouped_row(Z + (size_t)r * ldz, n_exp, n_groups, keep, top, scale, n_always, sel_idx + (size_t)r * tt, sel_w + (size_t)r * tt, rsm, rsm + n_exp,
                      rsm + 2 * n_exp, threadIdx.x);
}
// The router of the NEXT sublayer inside the residual update (few rows): what k_sandwich_add appends when it is given a router
struct GroupRouteNext {
    const bf16* w;             // [n_exp][ldw] router matrix, or null: no routing here
    int ldw, n_exp, n_groups, keep, top, n_always;
    float scale;
    int* sel_idx;              // [rows][top + n_always]
    float* sel_w;
};
// router logits of row r from the feed-forward's input sx [width] (shared memory; already rounded like the product's operand) -- a warp
// per output -- and the row's choices.  sx is followed by n_exp logits, 2 n_exp work floats and n_groups ranks.
__device__ __forceinline__ void sandwich_route(const GroupRouteNext& rn, float* sx, int width, int r) {
    float* sl = sx + width;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    for (int j = wid; j < rn.n_exp; j += nw) {
        const bf16* wr = rn.w + (size_t)j * rn.ldw;
        float a = 0.0f;
        const int w8 = width & ~7;                   // rows of the router matrix start on 16-byte boundaries: eight weights per load
        for (int c = lane * 8; c < w8; c += 256) {
            const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wr + c));
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                a = fmaf(sx[c + 2 * i], __uint_as_float(ww[i] << 16), a);
                a = fmaf(sx[c + 2 * i + 1], __uint_as_float(ww[i] & 0xffff0000u), a);
            }
        }
        for (int c = w8 + lane; c < width; c += 32) a = fmaf(sx[c], __bfloat162float(wr[c]), a);
        a = warp_sum(a);
        if (lane == 0) sl[j] = a;
    }
    __syncthreads();
    const int tt = rn.top + rn.n_always;
    if (wid == 0)
        route_grouped_row(sl, rn.n_exp, rn.n_groups, rn.keep, rn.top, rn.scale, rn.n_always, rn.sel_idx + (size_t)r * tt, rn.sel_w + (size_t)r * tt, sl + rn.n_exp,
                          sl + 2 * rn.n_exp, sl + 3 * rn.n_exp, lane);
}

// x = scale * embed[tok] and op = norm(x) in one kernel: the first layer's input (models without a bigram table)
template <typename OT>
__global__ void __launch_bounds__(256) k_embed_norm(PassTables t, const bf16* __restrict__ embed, int width, float scale, NormArgs nrm, float* __restrict__ x,
                                                    OT* __restrict__ op, int ld_op) {
    __shared__ float red[33];
    const int r = blockIdx.x, center = nrm.kind == SW_NORM_LAYER;
    const bf16* e = embed + (size_t)t.tok[r] * width;
    float* xr = x + (size_t)r * width;
    float s = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) { const float v = __bfloat162float(e[c]) * scale; xr[c] = v; s += v; }
    const float mean = center ? block_sum(s, red) / (float)width : 0.0f;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) { const float d = xr[c] - mean; ss += d * d; }      // a thread re-reads what it wrote
    const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)width + nrm.eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) op[(size_t)r * ld_op + c] = cvt<OT>((xr[c] - mean) * rstd * nrm.w[c] + (center ? nrm.b[c] : 0.0f));
}

// Residual update of the sandwich style: y = Y (+ Y2), or the sum of rows pair_dst[r * top + k] >= 0 of Yg (grouped experts, in order of k);
// x += post(y); when next.w is set, op = next(x) is the operand of the following matrix product.  Rows of up to 4 * SW_KEEP * 256 values
// stay in registers between the passes (16-byte accesses); wider or unaligned rows walk the row again.  With a router (rn.w; few rows) the
// kernel also forms the next sublayer's router logits from the operand row it has just written and picks the experts; dynamic shared
// memory: width + 3 n_exp + n_groups floats.
// SW_KEEP: float4 groups a thread keeps per array (1, 2 or 4: rows up to 1024, 2048, 4096 wide); fewer kept values, fewer registers, more rows
// in flight per SM -- the kernel is bound by the latency of a row's load / reduce / store chain, not by bandwidth.
template <typename OT, int SW_KEEP>
__global__ void __launch_bounds__(256, SW_KEEP == 4 ? 4 : SW_KEEP == 2 ? 6 : 8) k_sandwich_add(const float* __restrict__ Y, const float* __restrict__ Y2, const float* __restrict__ Yg,
                                                      const int* __restrict__ pair_dst, int top, int width, NormArgs post, float* __restrict__ x,
                                                      NormArgs next, OT* __restrict__ op, int ld_op, GroupRouteNext rn) {
    __shared__ float red[128];           // four reductions, each with 32 floats of its own (the walking path uses the first 33)
    __shared__ int sdst[PN_MAX_TOP];
    extern __shared__ float srt[];
    const int r = blockIdx.x;
    const int cp = post.kind == SW_NORM_LAYER, cn = next.kind == SW_NORM_LAYER;
    if (Yg && threadIdx.x < top) sdst[threadIdx.x] = pair_dst[(size_t)r * top + threadIdx.x];
    __syncthreads();
    float* xr = x + (size_t)r * width;
    if (width % 4 == 0 && width <= 4 * SW_KEEP * (int)blockDim.x && ld_op % 4 == 0) {
        float vy[4 * SW_KEEP], vx[4 * SW_KEEP];
#pragma unroll
        for (int i = 0; i < SW_KEEP; i++) {
            const int c = (threadIdx.x + i * blockDim.x) * 4;
            if (c < width) {
                float4 y = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (Y) y = *reinterpret_cast<const float4*>(Y + (size_t)r * width + c);
                if (Y2) { const float4 t4 = *reinterpret_cast<const float4*>(Y2 + (size_t)r * width + c); y.x += t4.x; y.y += t4.y; y.z += t4.z; y.w += t4.w; }
                if (Yg)
                    for (int k = 0; k < top; k++)
                        if (sdst[k] >= 0) { const float4 t4 = *reinterpret_cast<const float4*>(Yg + (size_t)sdst[k] * width + c); y.x += t4.x; y.y += t4.y; y.z += t4.z; y.w += t4.w; }
                const float4 xv = *reinterpret_cast<const float4*>(xr + c);
                vy[4 * i] = y.x; vy[4 * i + 1] = y.y; vy[4 * i + 2] = y.z; vy[4 * i + 3] = y.w;
                vx[4 * i] = xv.x; vx[4 * i + 1] = xv.y; vx[4 * i + 2] = xv.z; vx[4 * i + 3] = xv.w;
            }
        }
        float mean, rstd;
        sw_stats<SW_KEEP>(vy, width, cp, post.eps, red, mean, rstd);
#pragma unroll
        for (int i = 0; i < SW_KEEP; i++) {
            const int c = (threadIdx.x + i * blockDim.x) * 4;
            if (c < width) {
                const float4 w4 = *reinterpret_cast<const float4*>(post.w + c);
                const float4 b4 = cp ? *reinterpret_cast<const float4*>(post.b + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                vx[4 * i] += (vy[4 * i] - mean) * rstd * w4.x + b4.x; vx[4 * i + 1] += (vy[4 * i + 1] - mean) * rstd * w4.y + b4.y;
                vx[4 * i + 2] += (vy[4 * i + 2] - mean) * rstd * w4.z + b4.z; vx[4 * i + 3] += (vy[4 * i + 3] - mean) * rstd * w4.w + b4.w;
                *reinterpret_cast<float4*>(xr + c) = make_float4(vx[4 * i], vx[4 * i + 1], vx[4 * i + 2], vx[4 * i + 3]);
            }
        }
        if (!next.w) return;
        sw_stats<SW_KEEP>(vx, width, cn, next.eps, red + 64, mean, rstd);
#pragma unroll
        for (int i = 0; i < SW_KEEP; i++) {
            const int c = (threadIdx.x + i * blockDim.x) * 4;
            if (c < width) {
                const float4 w4 = *reinterpret_cast<const float4*>(next.w + c);
                const float4 b4 = cn ? *reinterpret_cast<const float4*>(next.b + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                const float h0 = (vx[4 * i] - mean) * rstd * w4.x + b4.x, h1 = (vx[4 * i + 1] - mean) * rstd * w4.y + b4.y;
                const float h2 = (vx[4 * i + 2] - mean) * rstd * w4.z + b4.z, h3 = (vx[4 * i + 3] - mean) * rstd * w4.w + b4.w;
                store4(op + (size_t)r * ld_op + c, h0, h1, h2, h3);
                if (rn.w) { srt[c] = ldf<OT>(op + (size_t)r * ld_op + c); srt[c + 1] = ldf<OT>(op + (size_t)r * ld_op + c + 1);      // as the product would read them
                            srt[c + 2] = ldf<OT>(op + (size_t)r * ld_op + c + 2); srt[c + 3] = ldf<OT>(op + (size_t)r * ld_op + c + 3); }
            }
        }
        if (rn.w) sandwich_route(rn, srt, width, r);
        return;
    }
    auto sub = [&](int c) {
        float a = Y ? Y[(size_t)r * width + c] : 0.0f;
        if (Y2) a += Y2[(size_t)r * width + c];
        if (Yg)
            for (int k = 0; k < top; k++)
                if (sdst[k] >= 0) a += Yg[(size_t)sdst[k] * width + c];
        return a;
    };
    float mean = 0.0f, s = 0.0f;
    if (cp) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) s += sub(c);
        mean = block_sum(s, red) / (float)width;
    }
    s = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) { const float d = sub(c) - mean; s += d * d; }
    float rstd = 1.0f / sqrtf(block_sum(s, red) / (float)width + post.eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) xr[c] += (sub(c) - mean) * rstd * post.w[c] + (cp ? post.b[c] : 0.0f);     // a thread re-reads only what it wrote
    if (!next.w) return;
    mean = 0.0f; s = 0.0f;
    if (cn) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) s += xr[c];
        mean = block_sum(s, red) / (float)width;
    }
    s = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) { const float d = xr[c] - mean; s += d * d; }
    rstd = 1.0f / sqrtf(block_sum(s, red) / (float)width + next.eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const OT h = cvt<OT>((xr[c] - mean) * rstd * next.w[c] + (cn ? next.b[c] : 0.0f));
        op[(size_t)r * ld_op + c] = h;
        if (rn.w) srt[c] = ldf<OT>(&h);
    }
    if (rn.w) sandwich_route(rn, srt, width, r);
}

// sc[r][0] = 1 / sqrt(mean(q_r^2) + eps) over the nq entries of row r's query projection, sc[r][1] the same for its nk key entries (nk may be 0)
__global__ void __launch_bounds__(256) k_proj_rms(const float* __restrict__ P, int ldp, int q_off, int nq, int k_off, int nk, float eps, float* __restrict__ sc) {
    __shared__ float red[33];
    const int r = blockIdx.x;
    const float* p = P + (size_t)r * ldp;
    float a = 0.0f, b = 0.0f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = p[q_off + i]; a += v * v; }
    for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = p[k_off + i]; b += v * v; }
    a = block_sum(a, red);
    b = block_sum(b, red);
    if (threadIdx.x == 0) {
        sc[(size_t)r * 2] = 1.0f / sqrtf(a / (float)nq + eps);
        sc[(size_t)r * 2 + 1] = nk > 0 ? 1.0f / sqrtf(b / (float)nk + eps) : 0.0f;
    }
}

// ------------------------------------------------------------------------------------------------ differential attention
struct DiffArgs {
    int heads, dim, vdim;
    float diff, eps, out_scale;
    const float *lq1, *lk1, *lq2, *lk2;     // [dim]
    int gate, g_off, a_off;                  // gate 0: none; 3: logistic of column g_off + head of P
};
// A [R][heads * 2 * vdim]: the two maps' outputs per head.  o = a1 - lambda a2, lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff;
// o / sqrt(mean(o^2) + eps) * (1 - diff), gate, weight -> operand.  A warp per (row, head).
template <typename OT>
__global__ void __launch_bounds__(128) k_diff_combine(DiffArgs b, const float* __restrict__ A, const float* __restrict__ P, int ldp, OT* __restrict__ out, int ld_out) {
    const int r = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float d1 = 0.0f, d2 = 0.0f;
    for (int i = lane; i < b.dim; i += 32) { d1 = fmaf(b.lq1[i], b.lk1[i], d1); d2 = fmaf(b.lq2[i], b.lk2[i], d2); }
    const float lambda = expf(warp_sum(d1)) - expf(warp_sum(d2)) + b.diff;
    for (int h = blockIdx.y * nw + wid; h < b.heads; h += gridDim.y * nw) {
        const float* a1 = A + ((size_t)r * b.heads + h) * 2 * b.vdim;
        const float* a2 = a1 + b.vdim;
        float ss = 0.0f;
        for (int i = lane; i < b.vdim; i += 32) { const float o = a1[i] - lambda * a2[i]; ss += o * o; }
        ss = warp_sum(ss);
        float sc = (1.0f - b.diff) * b.out_scale / sqrtf(ss / (float)b.vdim + b.eps);
        if (b.gate) sc *= sigmoidf_(P[(size_t)r * ldp + b.g_off + h]);
        for (int i = lane; i < b.vdim; i += 32) out[(size_t)r * ld_out + b.a_off + h * b.vdim + i] = cvt<OT>((a1[i] - lambda * a2[i]) * sc);
    }
}

// ------------------------------------------------------------------------------------------------ retention: activation, joint norm
// q, k, v <- silu(.) in place: columns [c0, c0 + n) of the projection buffer (q | k | v are neighbours)
__global__ void k_silu_cols(float* __restrict__ P, int ldp, int c0, int n, int R) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)R * n) return;
    float* p = P + (i / n) * ldp + c0 + (i % n);
    const float z = *p;
    *p = z * sigmoidf_(z);
}
// per row: o (all heads together) / sqrt(mean(o^2) + eps) * w, times the gate (1: silu, 2: logistic of P's column g_off + c), times out_scale
template <typename OT>
__global__ void __launch_bounds__(256) k_ret_post_all(RetBranch b, const float* __restrict__ w, const float* __restrict__ O, const float* __restrict__ P, int ldp,
                                                      OT* __restrict__ out, int ld_out) {
    __shared__ float red[33];
    const int r = blockIdx.x, n = b.heads * b.vdim;
    const float* o = O + (size_t)r * n;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) ss += o[c] * o[c];
    const float sc = b.out_scale / sqrtf(block_sum(ss, red) / (float)n + b.eps);
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        float v = o[c] * sc * w[c];
        if (b.gated) { const float g = P[(size_t)r * ldp + b.g_off + c]; v *= b.gated == 2 ? sigmoidf_(g) : g * sigmoidf_(g); }
        out[(size_t)r * ld_out + b.a_off + c] = cvt<OT>(v);
    }
}

}  // namespace seq
}  // namespace gtb
