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

// CTA = (segment, head); thread = (value column j, share `part` of KP key channels). The thread keeps its KP x 1 piece of the state in
// registers; a chunk of tokens' decays, keys, queries and values is staged in shared memory, every thread leaves its partial output per
// token there, and the shares are added once per chunk.
template <int KP>
__global__ void __launch_bounds__(1024) seq_gla_scan_kernel(sllm_seq_batch b, const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
                                                            const float* __restrict__ v, int ldv, const float* __restrict__ z, int ldz, int heads, int dk,
                                                            int dv, float qscale, float inv_tau, float* __restrict__ state, float* __restrict__ o,
                                                            int ldo, int chunk) {
    extern __shared__ float sm[];
    const int seg = blockIdx.x, h = blockIdx.y;
    const int dvp = (dv + 31) & ~31, parts = (dk + KP - 1) / KP;
    const int j = threadIdx.x % dvp, part = threadIdx.x / dvp;
    const bool live = j < dv && part < parts;
    float* s_al = sm;                   // [chunk][dk]
    float* s_k = s_al + chunk * dk;     // [chunk][dk]
    float* s_q = s_k + chunk * dk;      // [chunk][dk]
    float* s_v = s_q + chunk * dk;      // [chunk][dv]
    float* s_o = s_v + chunk * dv;      // [chunk][parts][dv]
    const int start = b.seg_start[seg], len = b.seg_len[seg], slot = b.seg_slot[seg];
    float* st = state + ((size_t)slot * heads + h) * dk * dv;
    float S[KP];
#pragma unroll
    for (int x = 0; x < KP; ++x) {
        const int kr = part * KP + x;
        S[x] = (live && kr < dk) ? st[(size_t)kr * dv + j] : 0.0f;
    }
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
                s_o[(i * parts + part) * dv + j] = acc;
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < n * dv; i += blockDim.x) {
            const int tok = i / dv, col = i % dv;
            float acc = 0.0f;
            for (int pp = 0; pp < parts; ++pp) acc += s_o[(tok * parts + pp) * dv + col];
            o[(size_t)(start + c0 + tok) * ldo + h * dv + col] = acc;
        }
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int x = 0; x < KP; ++x) {
            const int kr = part * KP + x;
            if (kr < dk) st[(size_t)kr * dv + j] = S[x];
        }
    }
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
                        int32_t ldo, sllm_stream_t stream) {
    if (int rc = check_segments(b, "seq_rglru_scan")) return rc;
    SLLM_REQUIRE(u && lr && li && ypre && lam && state && out && channels > 0, SLLM_EINVAL, "seq_rglru_scan: bad argument");
    SLLM_REQUIRE(taps >= 1 && taps <= kMaxTaps, SLLM_EINVAL, "seq_rglru_scan: 1..%d taps", kMaxTaps);
    seq_rglru_scan_kernel<<<dim3((channels + 63) / 64, b->nseg), 64, 0, as_stream(stream)>>>(*b, u, ldu, lr, li, ldg, ypre, ldy, lam, c, channels, state, xconv,
                                                                                              ldx, taps, tail, out, ldo);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_gla_scan(const sllm_seq_batch* b, const float* q, int32_t ldq, const float* k, int32_t ldk, const float* v, int32_t ldv, const float* z,
                      int32_t ldz, int32_t heads, int32_t dk, int32_t dv, float qscale, float tau, float* state, float* o, int32_t ldo, sllm_stream_t stream) {
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
if (smem > 48 * 1024) SLLM_CUDA(cudaFuncSetAttribute(seq_gla_scan_kernel<kp>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    seq_gla_scan_kernel<kp><<<grid, threads, smem, st>>>(*b, q, ldq, k, ldk, v, ldv, z, ldz, heads, dk, dv, qscale, 1.0f / tau, state, o, ldo, chunk);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

}  // extern "C"
