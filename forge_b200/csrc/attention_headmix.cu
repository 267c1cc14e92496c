// Attention whose heads exchange their weights after the softmax, over a sliding window that also keeps the
// first tokens of the sequence, on the paged cache; and the step that prepares its operands.
//
//   visible(i, j) = j <= i and (i - j < window or j < keep_first)            (window <= 0: every j <= i)
//   p_g(i, j)     = softmax over the visible j of  scale * q_g(i) . k_kv(g)(j)
//   w_h(i, j)     = sum_g mix[h, g] p_g(i, j)                                  (mix = null: w_h = p_h)
//   o_h(i)        = gate_h(i) * sum_j w_h(i, j) v_kv(h)(j)                     (gate = null: 1)
//
// Query/key heads have D channels and value heads E channels, which need not be equal; a cache page is
// [kv head][token in page][D] keys followed by [kv head][token in page][E] values (with D == E that is the
// layout [2, kv heads, page, D] of the other attention kernels).  All arithmetic is fp32 whatever the
// storage type.  Because a head's output needs every head's normalised weights, a tile of query tokens
// walks its keys twice: once for each (token, head)'s maximum and sum, once for weights, mixing and values.
// Keys are walked in chunks of KT positions that start at multiples of KT, so what a token adds up, and in
// which order, depends on its position alone: not on the step's cut, the tile, or the batch around it.
#include "common.cuh"
#include "checks.cuh"

namespace {

// One CTA per token: takes the fp32 result of the fused projection, row = [q heads | k heads | v heads | gates],
// rotates q and k (neighbouring channels 2i, 2i+1 form a pair, on the first rot_dims channels of a head, angle =
// position * inv_freq[i]), blends v with the same token's values of an earlier layer, v <- (1 - lam) v + lam v_first,
// stores q in the activation type and k, v at the token's cache slot, and turns the gate columns into sigmoids.
template <typename TC>
__global__ void __launch_bounds__(128)
headmix_prepare_kernel(const float* __restrict__ proj, int ld, const int32_t* __restrict__ positions,
                       const int32_t* __restrict__ slot_mapping, const float* __restrict__ inv_freq,
                       const float* __restrict__ v_first, const float* __restrict__ lam, float* __restrict__ v_keep,
                       TC* __restrict__ q_out, TC* __restrict__ cache, float* __restrict__ gate_out, int H, int G, int D,
                       int E, int rot_dims, int page_size, long long page_stride, int has_gate) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int t = blockIdx.x;
    const float* row = proj + (size_t)t * ld;
    const float pos = (float)positions[t];
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    const bool store = slot >= 0 && FORGE_SLOT_OK(slot);
    const int page = store ? slot / page_size : 0, off = store ? slot % page_size : 0;
    TC* kbase = cache + (size_t)page * page_stride;
    TC* vbase = kbase + (size_t)G * page_size * D;
    const int n_qk = (H + G) * D;
    const int first = blockIdx.y * blockDim.x + threadIdx.x, step = gridDim.y * blockDim.x;      // a row's work is spread over the CTAs of its grid row
    for (int idx = first; idx < n_qk; idx += step) {
        const int head = idx / D, d = idx % D;
        float x = row[idx];
        if (d < rot_dims) {
            float s, c;
            sincosf(pos * inv_freq[d >> 1], &s, &c);
            const float other = row[idx ^ 1];
            x = (d & 1) ? x * c + other * s : x * c - other * s;
        }
        if (head < H) q_out[(size_t)t * H * D + idx] = forge::from_float<TC>(x);
        else if (store) kbase[((size_t)(head - H) * page_size + off) * D + d] = forge::from_float<TC>(x);
    }
    const int n_v = G * E;
    const float l = (v_first && lam) ? lam[0] : 0.f;
    for (int idx = first; idx < n_v; idx += step) {
        float x = row[n_qk + idx];
        if (v_keep) v_keep[(size_t)t * n_v + idx] = x;
        if (v_first) x = (1.0f - l) * x + l * v_first[(size_t)t * n_v + idx];
        if (store) vbase[((size_t)(idx / E) * page_size + off) * E + idx % E] = forge::from_float<TC>(x);
    }
    if (has_gate)
        for (int h = first; h < H; h += step)
            gate_out[(size_t)t * H + h] = 1.0f / (1.0f + expf(-row[n_qk + n_v + h]));
}

__device__ __forceinline__ bool visible(int pos, int j, int window, int keep_first) {
    return j <= pos && (window <= 0 || pos - j < window || j < keep_first);
}

constexpr int kAttThreads = 256;

// One CTA per tile of up to TQ consecutive tokens of one request (tile_t0 = null: tile i is token i alone).
template <typename TC>
__global__ void __launch_bounds__(kAttThreads)
headmix_attention_kernel(const TC* __restrict__ q, const TC* __restrict__ cache, const int32_t* __restrict__ block_table,
                         const int32_t* __restrict__ tok_req, const int32_t* __restrict__ positions,
                         const int32_t* __restrict__ tile_t0, const int32_t* __restrict__ tile_n,
                         const float* __restrict__ mix, const float* __restrict__ gate, TC* __restrict__ out, int H, int G,
                         int D, int E, int page_size, long long page_stride, int max_pages, int window, int keep_first,
                         float scale, int TQ, int KT) {
    extern __shared__ float smem[];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int t0 = tile_t0 ? tile_t0[blockIdx.x] : blockIdx.x;
    const int nq = tile_n ? tile_n[blockIdx.x] : 1;
    if (!FORGE_TOKEN_OK(t0) || !FORGE_TOKEN_OK(t0 + nq - 1)) return;
    const int pos0 = positions[t0], pos_last = pos0 + nq - 1;
    const int32_t* table = block_table + (size_t)tok_req[t0] * max_pages;
    const int DP = D + 1, group = H / G;
    float* qs = smem;                       // [TQ][H][D]   queries, already scaled
    float* os = qs + TQ * H * D;            // [TQ][H][E]   outputs being added up
    float* ks = os + TQ * H * E;            // [G][KT][D+1] keys of the chunk
    float* vs = ks + G * KT * DP;           // [G][KT][E]   values of the chunk
    float* sc = vs + G * KT * E;            // [TQ][H][KT]  scores, then normalised weights
    float* pm = sc + TQ * H * KT;           // [TQ][H][KT]  weights after the heads' exchange
    float* ms = pm + TQ * H * KT;           // [TQ][H]      running maximum
    float* ls = ms + TQ * H;                // [TQ][H]      running sum
    float* mx = ls + TQ * H;                // [H][H]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = kAttThreads >> 5;

    for (int i = tid; i < nq * H * D; i += kAttThreads) qs[i] = forge::to_float(q[(size_t)t0 * H * D + i]) * scale;
    for (int i = tid; i < nq * H * E; i += kAttThreads) os[i] = 0.f;
    for (int i = tid; i < nq * H; i += kAttThreads) { ms[i] = -INFINITY; ls[i] = 0.f; }
    if (mix) for (int i = tid; i < H * H; i += kAttThreads) mx[i] = mix[i];

    // key positions that some token of the tile may see: the kept first ones below the window, and the window
    const int win_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int kept_hi = window > 0 ? min(keep_first, win_lo) : 0;
    const int kept_chunks = (kept_hi + KT - 1) / KT;
    const int first_win_chunk = max(kept_chunks, win_lo / KT), last_chunk = pos_last / KT;
    const int n_chunks = kept_chunks + (last_chunk - first_win_chunk + 1);

    for (int pass = 0; pass < 2; ++pass) {
        for (int ci = 0; ci < n_chunks; ++ci) {
            const int c = ci < kept_chunks ? ci : first_win_chunk + (ci - kept_chunks);
            const int j0 = c * KT;
            __syncthreads();                                  // the chunk before is done with ks, vs, sc, pm
            // keys (and in the second pass values) of positions j0 .. j0 + KT - 1; beyond the tile's last position: zeros
            for (int i = tid; i < G * KT * D; i += kAttThreads) {
                const int d = i % D, jj = (i / D) % KT, g = i / (D * KT);
                const int j = j0 + jj;
                float x = 0.f;
                if (j <= pos_last) {
                    const int page = table[j / page_size];
                    if (page >= 0 && FORGE_PAGE_OK(page))
                        x = forge::to_float(cache[(size_t)page * page_stride + ((size_t)g * page_size + j % page_size) * D + d]);
                }
                ks[(g * KT + jj) * DP + d] = x;
            }
            if (pass == 1) {
                for (int i = tid; i < G * KT * E; i += kAttThreads) {
                    const int e = i % E, jj = (i / E) % KT, g = i / (E * KT);
                    const int j = j0 + jj;
                    float x = 0.f;
                    if (j <= pos_last) {
                        const int page = table[j / page_size];
                        if (page >= 0 && FORGE_PAGE_OK(page))
                            x = forge::to_float(cache[(size_t)page * page_stride + (size_t)G * page_size * D +
                                                      ((size_t)g * page_size + j % page_size) * E + e]);
                    }
                    vs[i] = x;
                }
            }
            __syncthreads();
            // scores of every (token, head, key) of the chunk; -inf where the token does not see the key
            for (int i = tid; i < nq * H * KT; i += kAttThreads) {
                const int jj = i % KT, h = (i / KT) % H, tq = i / (KT * H);
                float s = -INFINITY;
                if (visible(pos0 + tq, j0 + jj, window, keep_first)) {
                    const float* qr = qs + (tq * H + h) * D;
                    const float* kr = ks + ((h / group) * KT + jj) * DP;
                    s = 0.f;
                    for (int d = 0; d < D; ++d) s = fmaf(qr[d], kr[d], s);
                }
                if (pass == 1) {
                    const float m = ms[tq * H + h];
                    s = s == -INFINITY ? 0.f : expf(s - m) / ls[tq * H + h];
                }
                sc[i] = s;
            }
            __syncthreads();
            if (pass == 0) {
                // a warp per (token, head): the chunk's maximum, then the running maximum and sum
                for (int r = warp; r < nq * H; r += nwarps) {
                    float cm = -INFINITY;
                    for (int jj = lane; jj < KT; jj += 32) cm = fmaxf(cm, sc[r * KT + jj]);
                    cm = forge::warp_max(cm);
                    if (cm == -INFINITY) continue;            // the token sees nothing of this chunk
                    const float m_old = ms[r], m_new = fmaxf(m_old, cm);
                    float sum = 0.f;
                    for (int jj = lane; jj < KT; jj += 32) sum += expf(sc[r * KT + jj] - m_new);
                    sum = forge::warp_sum(sum);
                    if (lane == 0) {
                        ls[r] = ls[r] * expf(m_old - m_new) + sum;
                        ms[r] = m_new;
                    }
                }
                continue;
            }
            const float* w = sc;
            if (mix) {
                for (int i = tid; i < nq * H * KT; i += kAttThreads) {
                    const int jj = i % KT, h = (i / KT) % H, tq = i / (KT * H);
                    float a = 0.f;
                    for (int g = 0; g < H; ++g) a = fmaf(mx[h * H + g], sc[(tq * H + g) * KT + jj], a);
                    pm[i] = a;
                }
                __syncthreads();
                w = pm;
            }
            for (int i = tid; i < nq * H * E; i += kAttThreads) {
                const int e = i % E, h = (i / E) % H, tq = i / (E * H);
                const float* wr = w + (tq * H + h) * KT;
                const float* vr = vs + (h / group) * KT * E + e;
                float a = 0.f;
                for (int jj = 0; jj < KT; ++jj) a = fmaf(wr[jj], vr[jj * E], a);
                os[i] += a;
            }
        }
    }
    __syncthreads();
    for (int i = tid; i < nq * H * E; i += kAttThreads) {
        const int h = (i / E) % H, tq = i / (E * H);
        const float g = gate ? gate[(size_t)(t0 + tq) * H + h] : 1.0f;
        out[(size_t)t0 * H * E + i] = forge::from_float<TC>(os[i] * g);
    }
}

size_t attention_smem_bytes(int H, int G, int D, int E, int TQ, int KT) {
    return sizeof(float) * ((size_t)TQ * H * (D + E) + (size_t)G * KT * (D + 1 + E) + 2 * (size_t)TQ * H * KT + 2 * (size_t)TQ * H +
                            (size_t)H * H);
}

forge::PerDeviceFlag g_attr_done[2];

}  // namespace

// proj fp32 [T, ld]: per row q heads (H x D), k heads (G x D), v heads (G x E), then H gate columns if has_gate.
// inv_freq fp32 [rot_dims / 2].  v_first / lam (both or neither): fp32 [T, G*E] and one fp32 number; v_keep: fp32
// [T, G*E] that receives the row's values before any blending, or null.  cache: pages of page_stride elements.
extern "C" int forge_headmix_prepare(const float* proj, int ld, const int32_t* positions, const int32_t* slot_mapping,
                                     const float* inv_freq, const float* v_first, const float* lam, float* v_keep, void* q_out,
                                     void* cache, float* gate_out, int dtype, int T, int H, int G, int D, int E, int rot_dims,
                                     int page_size, long long page_stride, int has_gate, cudaStream_t stream) {
    if (T < 0 || H <= 0 || G <= 0 || D <= 0 || E <= 0 || H % G != 0 || page_size <= 0 || rot_dims < 0 || rot_dims > D || (rot_dims & 1))
        return forge::fail(FORGE_ERR_ARG, "headmix_prepare: bad sizes T=%d H=%d G=%d D=%d E=%d rot=%d page=%d", T, H, G, D, E, rot_dims, page_size);
    if (ld < (H + G) * D + G * E + (has_gate ? H : 0)) return forge::fail(FORGE_ERR_ARG, "headmix_prepare: rows of %d are too short", ld);
    if (page_stride < (long long)G * page_size * (D + E)) return forge::fail(FORGE_ERR_ARG, "headmix_prepare: pages are too small");
    if ((v_first == nullptr) != (lam == nullptr)) return forge::fail(FORGE_ERR_ARG, "headmix_prepare: v_first and lam go together");
    if (has_gate && !gate_out) return forge::fail(FORGE_ERR_ARG, "headmix_prepare: no place for the gates");
    if (T == 0) return FORGE_OK;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(dtype, TT,
        e = forge::launch(headmix_prepare_kernel<TT>, dim3(T, T >= 256 ? 1 : ((H + G) * D + 511) / 512), dim3(128), 0, stream, 1, proj, ld, positions, slot_mapping, inv_freq,
                          v_first, lam, v_keep, (TT*)q_out, (TT*)cache, gate_out, H, G, D, E, rot_dims, page_size, page_stride, has_gate));
    return forge::check_launch("headmix_prepare", e);
}

// How many bytes of shared memory a tile of TQ tokens with key chunks of KT takes (the caller picks TQ and KT with it).
extern "C" long long forge_headmix_attention_smem(int H, int G, int D, int E, int TQ, int KT) {
    return (long long)attention_smem_bytes(H, G, D, E, TQ, KT);
}

// q, out in the cache's type: [T, H*D] and [T, H*E].  tile_t0 / tile_n int32 [num_tiles]: first token and number of
// tokens (<= TQ, consecutive, one request) of each tile; both null: num_tiles tiles of one token each.  mix fp32 [H, H]
// or null; gate fp32 [T, H] or null.  window <= 0: all earlier keys.
extern "C" int forge_headmix_attention(const void* q, const void* cache, const int32_t* block_table, const int32_t* tok_req,
                                       const int32_t* positions, const int32_t* tile_t0, const int32_t* tile_n, const float* mix,
                                       const float* gate, void* out, int dtype, int num_tiles, int H, int G, int D, int E,
                                       int page_size, long long page_stride, int max_pages, int window, int keep_first, float scale,
                                       int TQ, int KT, cudaStream_t stream) {
    if (num_tiles < 0 || H <= 0 || G <= 0 || D <= 0 || E <= 0 || H % G != 0 || page_size <= 0 || max_pages <= 0 || TQ <= 0 || KT <= 0 ||
        keep_first < 0)
        return forge::fail(FORGE_ERR_ARG, "headmix_attention: bad sizes tiles=%d H=%d G=%d D=%d E=%d page=%d TQ=%d KT=%d", num_tiles, H, G,
                           D, E, page_size, TQ, KT);
    if ((tile_t0 == nullptr) != (tile_n == nullptr)) return forge::fail(FORGE_ERR_ARG, "headmix_attention: half a tile list");
    if (num_tiles == 0) return FORGE_OK;
    const size_t smem = attention_smem_bytes(H, G, D, E, TQ, KT);
    if (smem > 200 * 1024) return forge::fail(FORGE_ERR_UNSUPPORTED, "headmix_attention: a tile of %d tokens and %d keys needs %zu bytes of shared memory", TQ, KT, smem);
    bool& done = g_attr_done[dtype == FORGE_BF16].current();
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(dtype, TT, {
        if (!done) {
            e = cudaFuncSetAttribute(headmix_attention_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return forge::check_launch("headmix_attention (shared memory)", e);
            done = true;
        }
        e = forge::launch(headmix_attention_kernel<TT>, dim3(num_tiles), dim3(kAttThreads), smem, stream, 1, (const TT*)q, (const TT*)cache,
                          block_table, tok_req, positions, tile_t0, tile_n, mix, gate, (TT*)out, H, G, D, E, page_size, page_stride,
                          max_pages, window, keep_first, scale, TQ, KT);
    });
    return forge::check_launch("headmix_attention", e);
}

FORGE_DEFINE_CHECKS_ENTRY(attention_headmix)
