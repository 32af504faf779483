// csrc/seq_recur.cu — recurrent layers of the ragged token batch: the short causal convolution and the real-gated linear recurrent unit
// of a Griffin-style recurrent block, and gated linear attention with a decay per key channel. Each sequence's state lives in a slot of
// an fp32 array and is carried from step to step; everything that enters a recurrence (gates, decays and their logarithms, the state) is
// fp32. A segment of the batch (a portion of a prompt or one decoded token) is walked token by token by the threads that own its state.
#include "seq_common.cuh"

namespace sllm {

// thread = (token, channel); the taps-1 inputs before a segment come from the sequence's tail
__global__ void seq_conv_kernel(sllm_seq_batch b, const float* __restrict__ x, int ldx, int channels, int taps, const float* __restrict__ w,
                                const float* __restrict__ cb, const float* __restrict__ tail, float* __restrict__ u, int ldu) {
    const int t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int slot = b.tok_slot[t];
    float acc = cb ? cb[c] : 0.0f;
    acc = fmaf(w[(size_t)c * taps + taps - 1], x[(size_t)t * ldx + c], acc);
    int in_batch = 1;   // are the predecessors still inside this step's portion?
    for (int back = 1; back < taps; ++back) {
        float xv;
        if (in_batch && t - back >= 0 && b.tok_slot[t - back] == slot) {
            xv = x[(size_t)(t - back) * ldx + c];
        } else {
            // `back - 1` predecessors were found in the batch up to here or earlier; the first miss fixes the offset in the segment
            if (in_batch) in_batch = 0;
            int i = 0;
            while (i < back && t - 1 - i >= 0 && b.tok_slot[t - 1 - i] == slot) ++i;   // tokens of this segment in front of t
            xv = tail ? tail[((size_t)slot * (taps - 1) + (taps - 1 + i - back)) * channels + c] : 0.0f;
        }
        acc = fmaf(w[(size_t)c * taps + taps - 1 - back], xv, acc);
    }
    u[(size_t)t * ldu + c] = acc;
}

constexpr int kMaxTaps = 16;

// thread = (segment, channel)
__global__ void seq_rglru_scan_kernel(sllm_seq_batch b, const float* __restrict__ u, int ldu, const float* __restrict__ lr, const float* __restrict__ li,
                                      int ldg, const float* __restrict__ ypre, int ldy, const float* __restrict__ lam, float cc, int channels,
                                      float* __restrict__ state, const float* __restrict__ xconv, int ldx, int taps, float* __restrict__ tail,
                                      float* __restrict__ out, int ldo) {
    const int seg = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int start = b.seg_start[seg], len = b.seg_len[seg], slot = b.seg_slot[seg];
    // The state is carried in double INSIDE a portion and stored as fp32 between steps. A decay close to 1 (long memory) is not
    // representable in fp32 better than to 6e-8, and that rounding, applied once per token, adds up over the channel's memory length:
    // after a thousand tokens the fp32 recurrence is off by 2e-6 of the state. exp / expm1 of the fp32 logarithm in double keep it exact.
    double S = (double)state[(size_t)slot * channels + c];
    const float sp = seq_softplus(lam[c]);
    for (int i = 0; i < len; ++i) {
        const size_t t = (size_t)(start + i);
        const float r = seq_sigmoid(lr[t * ldg + c]), ig = seq_sigmoid(li[t * ldg + c]);
        const float la = -cc * r * sp;               // log of the decay
        const double a = exp((double)la);
        const double mult = sqrt(-expm1(2.0 * (double)la));   // sqrt(1 - a^2) without cancellation near a = 1
        S = fma(a, S, mult * (double)(ig * u[t * ldu + c]));
        out[t * ldo + c] = (float)S * seq_gelu_tanh(ypre[t * ldy + c]);
    }
    state[(size_t)slot * channels + c] = (float)S;
    if (xconv && tail && taps > 1) {
        float keep[kMaxTaps];
        const int n = taps - 1;
        for (int r = 0; r < n; ++r) {
            const int idx = len + r - n;   // row of the segment that lands in tail row r (negative: still an old tail row)
            keep[r] = idx >= 0 ? xconv[(size_t)(start + idx) * ldx + c] : tail[((size_t)slot * n + (r + len)) * channels + c];
        }
        for (int r = 0; r < n; ++r) tail[((size_t)slot * n + r) * channels + c] = keep[r];
    }
}

// ---- the same recurrence for long portions: three passes over tiles of 32 tokens -------------------------------------------------------
// S_t = a_t S_(t-1) + b_t is linear in S, so a tile's effect on the state is (P, Q): S_end = P * S_start + Q with P = prod a_t and
// Q = the tile's result from a zero state. Pass 1 computes (P, Q) of every tile in parallel, pass 2 walks each sequence's tiles in order
// (one fused multiply-add per tile and channel) and leaves every tile's start state, pass 3 redoes the tiles from their start states and
// writes the outputs. The token loop of a 2048-token portion becomes 32 + 64 + 32 dependent steps instead of 2048.
struct RgTile {
    int start, n, cid, seg;
};
__device__ __forceinline__ RgTile rg_tile(const sllm_seq_batch& b, int tile) {
    RgTile r;
    r.seg = b.qt_seg[tile];
    const int off = b.qt_off[tile];
    r.start = b.seg_start[r.seg] + off;
    r.n = min(32, b.seg_len[r.seg] - off);
    r.cid = b.seg_tile0[r.seg] + off / 32;
    return r;
}
__device__ __forceinline__ void rg_coeffs(float lr, float li, float uu, float sp, float cc, double* a, double* bb) {
    const float r = seq_sigmoid(lr), ig = seq_sigmoid(li);
    const float la = -cc * r * sp;
    *a = exp((double)la);
    *bb = sqrt(-expm1(2.0 * (double)la)) * (double)(ig * uu);
}

// thread = (tile, channel)
__global__ void seq_rglru_tile_kernel(sllm_seq_batch b, const float* __restrict__ u, int ldu, const float* __restrict__ lr, const float* __restrict__ li,
                                      int ldg, const float* __restrict__ lam, float cc, int channels, double* __restrict__ PQ) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const RgTile tl = rg_tile(b, blockIdx.y);
    const float sp = seq_softplus(lam[c]);
    double P = 1.0, Q = 0.0;
    for (int i = 0; i < tl.n; ++i) {
        const size_t t = (size_t)(tl.start + i);
        double a, bb;
        rg_coeffs(lr[t * ldg + c], li[t * ldg + c], u[t * ldu + c], sp, cc, &a, &bb);
        Q = fma(a, Q, bb);
        P *= a;
    }
    PQ[((size_t)tl.cid * 2) * channels + c] = P;
    PQ[((size_t)tl.cid * 2 + 1) * channels + c] = Q;
}

// thread = (segment, channel): the tiles of the segment in order; PQ[cid][0] becomes the tile's start state
__global__ void seq_rglru_carry_kernel(sllm_seq_batch b, int channels, double* __restrict__ PQ, float* __restrict__ state, const float* __restrict__ xconv,
                                       int ldx, int taps, float* __restrict__ tail) {
    const int seg = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int start = b.seg_start[seg], len = b.seg_len[seg], slot = b.seg_slot[seg], cid0 = b.seg_tile0[seg];
    double S = (double)state[(size_t)slot * channels + c];
    const int tiles = (len + 31) / 32;
#pragma unroll 4
    for (int k = 0; k < tiles; ++k) {
        const size_t at = ((size_t)(cid0 + k) * 2) * channels + c;
        const double P = PQ[at], Q = PQ[at + channels];
        PQ[at] = S;
        S = fma(P, S, Q);
    }
    state[(size_t)slot * channels + c] = (float)S;
    if (xconv && tail && taps > 1) {
        float keep[kMaxTaps];
        const int n = taps - 1;
        for (int r = 0; r < n; ++r) {
            const int idx = len + r - n;
            keep[r] = idx >= 0 ? xconv[(size_t)(start + idx) * ldx + c] : tail[((size_t)slot * n + (r + len)) * channels + c];
        }
        for (int r = 0; r < n; ++r) tail[((size_t)slot * n + r) * channels + c] = keep[r];
    }
}

// thread = (tile, channel): the tile again from its start state, outputs written
__global__ void seq_rglru_emit_kernel(sllm_seq_batch b, const float* __restrict__ u, int ldu, const float* __restrict__ lr, const float* __restrict__ li,
                                      int ldg, const float* __restrict__ ypre, int ldy, const float* __restrict__ lam, float cc, int channels,
                                      const double* __restrict__ PQ, float* __restrict__ out, int ldo) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const RgTile tl = rg_tile(b, blockIdx.y);
    const float sp = seq_softplus(lam[c]);
    double S = PQ[((size_t)tl.cid * 2) * channels + c];
    for (int i = 0; i < tl.n; ++i) {
        const size_t t = (size_t)(tl.start + i);
        double a, bb;
        rg_coeffs(lr[t * ldg + c], li[t * ldg + c], u[t * ldu + c], sp, cc, &a, &bb);
        S = fma(a, S, bb);
        out[t * ldo + c] = (float)S * seq_gelu_tanh(ypre[t * ldy + c]);
    }
}

// CTA = (segment, head); thread = (value column j, share `part` of KP key channels). The thread keeps its KP x 1 piece of the state in
// registers; a chunk of tokens' decays, keys, queries and values is staged in shared memory, every thread leaves its partial output per
// token there, and the shares are added once per chunk.
// MODE 0: a CTA walks a whole segment from the sequence's state and stores the state back (short portions, decoding).
// MODE 1 / 2: the three-pass form for long portions, as for the recurrent unit above, per tile of 32 tokens: pass 1 starts from zero and
// leaves the tile's (P = product of the decays per key channel, Q = its state) in `pbuf` / `qbuf`; seq_gla_carry_kernel turns Q into the
// tile's start state; pass 2 redoes the tile from there and writes the outputs.
template <int KP, int MODE>
__global__ void __launch_bounds__(1024) seq_gla_scan_kernel(sllm_seq_batch b, const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
                                                            const float* __restrict__ v, int ldv, const float* __restrict__ z, int ldz, int heads, int dk,
                                                            int dv, float qscale, float inv_tau, float* __restrict__ state, float* __restrict__ o,
                                                            int ldo, int chunk, float* __restrict__ pbuf, float* __restrict__ qbuf) {
    extern __shared__ float sm[];
    const int h = blockIdx.y;
    int seg, start, len, cid = 0;
    if (MODE == 0) {
        seg = blockIdx.x;
        start = b.seg_start[seg];
        len = b.seg_len[seg];
    } else {
        seg = b.qt_seg[blockIdx.x];
        const int off = b.qt_off[blockIdx.x];
        start = b.seg_start[seg] + off;
        len = min(32, b.seg_len[seg] - off);
        cid = b.seg_tile0[seg] + off / 32;
    }
    const int dvp = (dv + 31) & ~31, parts = (dk + KP - 1) / KP;
    const int j = threadIdx.x % dvp, part = threadIdx.x / dvp;
    const bool live = j < dv && part < parts;
    float* s_al = sm;                   // [chunk][dk]
    float* s_k = s_al + chunk * dk;     // [chunk][dk]
    float* s_q = s_k + chunk * dk;      // [chunk][dk]
    float* s_v = s_q + chunk * dk;      // [chunk][dv]
    float* s_o = s_v + chunk * dv;      // [chunk][parts][dv]
    const int slot = b.seg_slot[seg];
    float* st = MODE == 0 ? state + ((size_t)slot * heads + h) * dk * dv : qbuf + ((size_t)cid * heads + h) * dk * dv;
    float S[KP];
#pragma unroll
    for (int x = 0; x < KP; ++x) {
        const int kr = part * KP + x;
        S[x] = (MODE != 1 && live && kr < dk) ? st[(size_t)kr * dv + j] : 0.0f;
    }
    float pprod = 1.0f;   // MODE 1: product of this tile's decays of key channel threadIdx.x
    for (int c0 = 0; c0 < len; c0 += chunk) {
        const int n = min(chunk, len - c0);
        for (int i = threadIdx.x; i < n * dk; i += blockDim.x) {
            const size_t t = (size_t)(start + c0 + i / dk);
            const int col = h * dk + i % dk;
            // alpha = sigmoid(z)^(1/tau) = exp(-softplus(-z) / tau)
            s_al[i] = expf(-seq_softplus(-z[t * ldz + col]) * inv_tau);
            s_k[i] = k[t * ldk + col];
            s_q[i] = q[t * ldq + col] * qscale;
        }
        for (int i = threadIdx.x; i < n * dv; i += blockDim.x) s_v[i] = v[(size_t)(start + c0 + i / dv) * ldv + h * dv + i % dv];
        __syncthreads();
        if (MODE == 1 && threadIdx.x < dk)
            for (int i = 0; i < n; ++i) pprod *= s_al[i * dk + threadIdx.x];
        if (live) {
            for (int i = 0; i < n; ++i) {
                const float vj = s_v[i * dv + j];
                const float *al = s_al + i * dk + part * KP, *kk = s_k + i * dk + part * KP, *qq = s_q + i * dk + part * KP;
                float acc = 0.0f;
#pragma unroll
                for (int x = 0; x < KP; ++x) {
                    if (part * KP + x < dk) {
                        S[x] = fmaf(al[x], S[x], kk[x] * vj);
                        acc = fmaf(S[x], qq[x], acc);
                    }
                }
                if (MODE != 1) s_o[(i * parts + part) * dv + j] = acc;
            }
        }
        __syncthreads();
        if (MODE != 1)
        for (int i = threadIdx.x; i < n * dv; i += blockDim.x) {
            const int tok = i / dv, col = i % dv;
            float acc = 0.0f;
            for (int pp = 0; pp < parts; ++pp) acc += s_o[(tok * parts + pp) * dv + col];
            o[(size_t)(start + c0 + tok) * ldo + h * dv + col] = acc;
        }
        __syncthreads();
    }
    if (MODE != 2 && live) {
#pragma unroll
        for (int x = 0; x < KP; ++x) {
            const int kr = part * KP + x;
            if (kr < dk) st[(size_t)kr * dv + j] = S[x];
        }
    }
    if (MODE == 1 && threadIdx.x < dk) pbuf[((size_t)cid * heads + h) * dk + threadIdx.x] = pprod;
}

// thread = one element (key channel, value column) of one head's state of one segment: the segment's tiles in order, Q -> start state
__global__ void seq_gla_carry_kernel(sllm_seq_batch b, int heads, int dk, int dv, const float* __restrict__ pbuf, float* __restrict__ qbuf,
                                     float* __restrict__ state) {
    const int seg = blockIdx.z, h = blockIdx.y, e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= dk * dv) return;
    const int kr = e / dv;
    const int len = b.seg_len[seg], slot = b.seg_slot[seg], cid0 = b.seg_tile0[seg], tiles = (len + 31) / 32;
    float* sp = state + ((size_t)slot * heads + h) * dk * dv + e;
    float S = *sp;
#pragma unroll 4
    for (int k = 0; k < tiles; ++k) {
        const float P = pbuf[((size_t)(cid0 + k) * heads + h) * dk + kr];
        float* qp = qbuf + ((size_t)(cid0 + k) * heads + h) * dk * dv + e;
        const float Q = *qp;
        *qp = S;
        S = fmaf(P, S, Q);
    }
    *sp = S;
}

}  // namespace sllm

using namespace sllm;

static int check_segments(const sllm_seq_batch* b, const char* who) {
    SLLM_REQUIRE(b && b->T > 0 && b->nseg > 0 && b->tok_slot && b->tok_pos && b->seg_start && b->seg_len && b->seg_slot && b->seg_pos0, SLLM_EINVAL,
                 "%s: incomplete batch description", who);
    return SLLM_OK;
}

extern "C" {

int sllm_seq_conv(const sllm_seq_batch* b, const float* x, int32_t ldx, int32_t channels, int32_t taps, const float* w, const float* cb, const float* tail,
                  float* u, int32_t ldu, sllm_stream_t stream) {
    if (int rc = check_segments(b, "seq_conv")) return rc;
    SLLM_REQUIRE(x && w && u && channels > 0 && taps >= 1 && taps <= kMaxTaps, SLLM_EINVAL, "seq_conv: bad argument (1..%d taps)", kMaxTaps);
    SLLM_REQUIRE(taps == 1 || tail, SLLM_EINVAL, "seq_conv: a convolution over more than one tap needs the sequences' tails");
    SLLM_REQUIRE(b->T <= 65535, SLLM_ENOTSUP, "seq_conv: at most 65535 tokens per step");
    seq_conv_kernel<<<dim3((channels + 127) / 128, b->T), 128, 0, as_stream(stream)>>>(*b, x, ldx, channels, taps, w, cb, tail, u, ldu);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_rglru_scan(const sllm_seq_batch* b, const float* u, int32_t ldu, const float* lr, const float* li, int32_t ldg, const float* ypre, int32_t ldy,
                        const float* lam, float c, int32_t channels, float* state, const float* xconv, int32_t ldx, int32_t taps, float* tail, float* out,
                        int32_t ldo, void* scratch, sllm_stream_t stream) {
    if (int rc = check_segments(b, "seq_rglru_scan")) return rc;
    SLLM_REQUIRE(u && lr && li && ypre && lam && state && out && channels > 0, SLLM_EINVAL, "seq_rglru_scan: bad argument");
    SLLM_REQUIRE(taps >= 1 && taps <= kMaxTaps, SLLM_EINVAL, "seq_rglru_scan: 1..%d taps", kMaxTaps);
    if (scratch && b->n_qtiles > b->nseg && b->qt_seg && b->qt_off && b->seg_tile0) {   // some portion is longer than a tile: three passes
        double* PQ = reinterpret_cast<double*>(scratch);
        const dim3 tiles((channels + 127) / 128, b->n_qtiles), segs((channels + 127) / 128, b->nseg);
        seq_rglru_tile_kernel<<<tiles, 128, 0, as_stream(stream)>>>(*b, u, ldu, lr, li, ldg, lam, c, channels, PQ);
        seq_rglru_carry_kernel<<<segs, 128, 0, as_stream(stream)>>>(*b, channels, PQ, state, xconv, ldx, taps, tail);
        seq_rglru_emit_kernel<<<tiles, 128, 0, as_stream(stream)>>>(*b, u, ldu, lr, li, ldg, ypre, ldy, lam, c, channels, PQ, out, ldo);
        g_launches += 3;
        SLLM_LAUNCH_CHECK();
        return SLLM_OK;
    }
    seq_rglru_scan_kernel<<<dim3((channels + 63) / 64, b->nseg), 64, 0, as_stream(stream)>>>(*b, u, ldu, lr, li, ldg, ypre, ldy, lam, c, channels, state, xconv,
                                                                                              ldx, taps, tail, out, ldo);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_gla_scan(const sllm_seq_batch* b, const float* q, int32_t ldq, const float* k, int32_t ldk, const float* v, int32_t ldv, const float* z,
                      int32_t ldz, int32_t heads, int32_t dk, int32_t dv, float qscale, float tau, float* state, float* o, int32_t ldo, void* scratch, sllm_stream_t stream) {
    if (int rc = check_segments(b, "seq_gla_scan")) return rc;
    SLLM_REQUIRE(q && k && v && z && state && o && heads > 0 && dk > 0 && dv > 0 && tau > 0.0f, SLLM_EINVAL, "seq_gla_scan: bad argument");
    const int dvp = (dv + 31) & ~31;
    SLLM_REQUIRE(dvp <= 1024, SLLM_ENOTSUP, "seq_gla_scan: value width %d beyond 1024", dv);
    constexpr int kp = 32;   // key channels per thread: 32 state registers; a head needs dvp * ceil(dk / 32) <= 1024 threads
    const int parts = (dk + kp - 1) / kp;
    SLLM_REQUIRE(dvp * parts <= 1024, SLLM_ENOTSUP, "seq_gla_scan: a %d x %d state does not fit one thread block (dk/32 * dv <= 1024)", dk, dv);
    const int per_tok = 3 * dk + dv + parts * dv;
    const int chunk = std::max(1, std::min(16, 10240 / per_tok));
    const size_t smem = (size_t)chunk * per_tok * sizeof(float);
    SLLM_REQUIRE(smem <= (size_t)smem_optin_bytes(), SLLM_ENOTSUP, "seq_gla_scan: one token of a %d x %d head needs %zu bytes of shared memory", dk, dv, smem);
    dim3 grid(b->nseg, heads);
    const int threads = dvp * parts;
    cudaStream_t st = as_stream(stream);
if (smem > 48 * 1024) {
        SLLM_CUDA(cudaFuncSetAttribute(seq_gla_scan_kernel<kp, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        SLLM_CUDA(cudaFuncSetAttribute(seq_gla_scan_kernel<kp, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        SLLM_CUDA(cudaFuncSetAttribute(seq_gla_scan_kernel<kp, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
    if (scratch && b->n_qtiles > b->nseg && b->qt_seg && b->qt_off && b->seg_tile0) {   // some portion is longer than a tile: three passes
        float* pbuf = reinterpret_cast<float*>(scratch);
        float* qbuf = pbuf + (((size_t)b->n_qtiles * heads * dk + 63) / 64) * 64;
        const dim3 tiles(b->n_qtiles, heads);
        seq_gla_scan_kernel<kp, 1><<<tiles, threads, smem, st>>>(*b, q, ldq, k, ldk, v, ldv, z, ldz, heads, dk, dv, qscale, 1.0f / tau, state, o, ldo, chunk,
                                                                   pbuf, qbuf);
        seq_gla_carry_kernel<<<dim3((dk * dv + 255) / 256, heads, b->nseg), 256, 0, st>>>(*b, heads, dk, dv, pbuf, qbuf, state);
        seq_gla_scan_kernel<kp, 2><<<tiles, threads, smem, st>>>(*b, q, ldq, k, ldk, v, ldv, z, ldz, heads, dk, dv, qscale, 1.0f / tau, state, o, ldo, chunk,
                                                                   pbuf, qbuf);
        g_launches += 3;
        SLLM_LAUNCH_CHECK();
        return SLLM_OK;
    }
    seq_gla_scan_kernel<kp, 0><<<grid, threads, smem, st>>>(*b, q, ldq, k, ldk, v, ldv, z, ldz, heads, dk, dv, qscale, 1.0f / tau, state, o, ldo, chunk,
                                                              nullptr, nullptr);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

}  // extern "C"
