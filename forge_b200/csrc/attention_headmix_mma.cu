// Tensor-core form (bf16 operands, fp32 sums) of the attention whose heads exchange their weights after the softmax,
// for prompt portions and single tokens alike; see attention_headmix.cu for the definition and the cache layout.
//
// The exchange  w_h = sum_g mix[h, g] p_g  is linear, so it can be taken after the values:
//     o_h(i) = gate_h(i) * sum_g mix[h, g] * ( p_g(i, .) V_kv(h) )
// The first kernel is therefore an ordinary one-pass attention per head g (running maximum and sum, nothing to meet
// between heads) whose value matrix is ALL key/value heads' values side by side, G*E columns: it leaves, normalised,
// u[i, g, :] = p_g(i, .) [V_0 | V_1 | ... ] in fp32.  The second kernel takes the sum over g for every head h from the
// columns of h's own key/value head and applies the gate.  The price is G times the value product of an attention
// without the exchange; what it buys is that no head waits for another and the weights never leave the registers.
//
// A CTA of four warps takes a tile of up to 64 rows = tokens x the query heads of ONE key/value head (consecutive
// tokens of one request; a single token brings H/G rows), one chunk of VC value columns, and walks the keys in tiles
// of 64 positions that start at multiples of 64: first the kept first positions below the window, then the window.
// mma.sync m16n8k16 (the legacy tensor path): S = Q K^T with K rows as the column-major operand, O += P V with V
// through ldmatrix.trans.
#include "common.cuh"
#include "checks.cuh"

namespace {

constexpr int BM = 64, BN = 64, kThreads = 128, kPad = 8;
constexpr int kMmaSmemLimit = 200 * 1024;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16 bytes from global to shared memory without a stop in registers; ok == false writes zeros instead
__device__ __forceinline__ void copy16_async(void* dst, const void* src, bool ok) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = ok ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ float ex2(float x) {          // 2^x, relative error 2^-22; ex2(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ bool visible(int pos, int j, int window, int keep_first) {
    return j <= pos && (window <= 0 || pos - j < window || j < keep_first);
}

// u fp32 [T, H, GE] (GE = G*E): u[t, g, :] = softmax_j(scale q_g(t) . k_kv(g)(j)) [v_0(j) | ... | v_{G-1}(j)].
template <int VC>
__global__ void __launch_bounds__(kThreads)
headmix_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache, const int32_t* __restrict__ block_table,
                   const int32_t* __restrict__ tok_req, const int32_t* __restrict__ positions, const int32_t* __restrict__ tile_t0,
                   const int32_t* __restrict__ tile_n, float* __restrict__ u, float* __restrict__ part_ml, int nsplit, int nstages, int qrows, int T, int H,
                   int G, int D, int E, int page_size, long long page_stride, int max_pages, int window, int keep_first, float scale) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int tile = blockIdx.x / nsplit, sp = blockIdx.x % nsplit, c = blockIdx.y, v0 = blockIdx.z * VC;
    const int t0 = tile_t0 ? tile_t0[tile] : tile;
    const int nq = tile_n ? tile_n[tile] : 1;
    if (!FORGE_TOKEN_OK(t0) || !FORGE_TOKEN_OK(t0 + nq - 1)) return;
    const int Gq = H / G, rows = nq * Gq, GE = G * E;
    const int pos0 = positions[t0], pos_last = pos0 + nq - 1;
    const int32_t* table = block_table + (size_t)tok_req[t0] * max_pages;
    const int DP = D + kPad, VP = VC + kPad;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [BM][D + 8]
    const int stage = BN * (DP + VP);                                     // elements of one buffer: a key tile and a value tile
    __nv_bfloat16* Ks = Qs + qrows * DP;                                  // nstages x [BN][D + 8]   (qrows: 64, or 16 for single tokens)
    __nv_bfloat16* Vs = Ks + BN * DP;                                     // nstages x [BN][VC + 8], each behind its key tile
    __shared__ int voff[VC / 8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint4 zero4 = make_uint4(0, 0, 0, 0);

    // queries: row r = token t0 + r / Gq, head c * Gq + r % Gq
    const int dchunks = D >> 3;
    for (int i = tid; i < qrows * dchunks; i += kThreads) {
        const int r = i / dchunks, ch = i % dchunks;
        uint4 val = zero4;
        if (r < rows)
            val = *reinterpret_cast<const uint4*>(q + ((size_t)(t0 + r / Gq) * H + c * Gq + r % Gq) * D + ch * 8);
        *reinterpret_cast<uint4*>(Qs + r * DP + ch * 8) = val;
    }

    float oacc[VC / 8][4];
#pragma unroll
    for (int i = 0; i < VC / 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
    float row_m[2] = {-INFINITY, -INFINITY}, row_l[2] = {0.f, 0.f};
    // A tile of at most 16 rows (a single token: H/G rows) would leave three warps idle: there all four warps take the same
    // 16 rows, each computes the scores again, and each takes a quarter of the value columns.
    const bool colsplit = rows <= 16;
    const int rb = colsplit ? 0 : warp;                                   // this warp's block of 16 rows
    const int ntw = colsplit ? VC / 32 : VC / 8, cb = colsplit ? warp * (VC / 4) : 0;     // its value columns: ntw blocks of 8 from cb
    const int r_lo = rb * 16 + (lane >> 2), r_hi = r_lo + 8;             // this thread's two rows
    const int pos_lo = pos0 + min(r_lo, rows - 1) / Gq, pos_hi = pos0 + min(r_hi, rows - 1) / Gq;
    const bool live_lo = r_lo < rows, live_hi = r_hi < rows;

    const int win_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int kept_hi = window > 0 ? min(keep_first, win_lo) : 0;
    const int kept_tiles = (kept_hi + BN - 1) / BN;
    const int first_win_tile = max(kept_tiles, win_lo / BN), last_tile = pos_last / BN;
    const int n_tiles = kept_tiles + (last_tile - first_win_tile + 1);
    const float sl2 = scale * 1.4426950408889634f;                        // scores in units of log2(e)
    const int vchunks = VC >> 3;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    if (tid < vchunks) {
        const int col = v0 + tid * 8;
        voff[tid] = col < GE ? G * page_size * D + (col / E) * page_size * E + col % E : -1;
    }
    __syncthreads();

    // key and value tiles go through two buffers: tile ti + 1 is on its way while tile ti is worked on
    // Two threads a key row: one look into the block table per thread and tile; what depends on the column alone (which
    // key/value head a 16-byte piece of a value row belongs to, and where in it) was worked out once, into voff.
    const int frow = tid >> 1, fpar = tid & 1;
    auto fetch = [&](int ti, int buf) {
        const int kt = ti < kept_tiles ? ti : first_win_tile + (ti - kept_tiles);
        const int j = kt * BN + frow;
        __nv_bfloat16* Kb = Ks + buf * stage + frow * DP;
        __nv_bfloat16* Vb = Vs + buf * stage + frow * VP;
        const __nv_bfloat16* page_base = cache;
        bool ok = false;
        if (j <= pos_last) {
            const int page = table[j >> page_shift];
            if (page >= 0 && FORGE_PAGE_OK(page)) {
                ok = true;
                page_base = cache + (size_t)page * page_stride;
            }
        }
        const int off = j & (page_size - 1);
        const __nv_bfloat16* ksrc = page_base + ((size_t)c * page_size + off) * D;
        for (int ch = fpar; ch < dchunks; ch += 2) copy16_async(Kb + ch * 8, ok ? ksrc + ch * 8 : cache, ok);
        const __nv_bfloat16* vsrc = page_base + (size_t)off * E;
        for (int ch = fpar; ch < vchunks; ch += 2) {
            const int o = voff[ch];
            copy16_async(Vb + ch * 8, (ok && o >= 0) ? vsrc + o : cache, ok && o >= 0);
        }
        copies_commit();
    };
    // nsplit > 1 (steps of single tokens): the key tiles are dealt out to nsplit CTAs in runs; each leaves its sums as they
    // are, with the row's maximum and sum, and the second kernel puts the runs together
    const int per = (n_tiles + nsplit - 1) / nsplit, ti_lo = sp * per, ti_hi = min(n_tiles, ti_lo + per);
    // nstages buffers: tiles ti + 1 .. ti + nstages - 1 are on their way while tile ti is worked on (two for prompt portions,
    // whose tiles are long work; more for single tokens, where a tile is little work and a copy's latency is what counts).
    // A group of copies is committed per tile, an empty one past the end, so that "all but the newest nstages - 1" always
    // means that tile ti has landed.
    for (int p = 0; p < nstages - 1; ++p) {
        if (ti_lo + p < ti_hi) fetch(ti_lo + p, p);
        else copies_commit();
    }
    for (int ti = ti_lo; ti < ti_hi; ++ti) {
        const int kt = ti < kept_tiles ? ti : first_win_tile + (ti - kept_tiles);
        const int j0 = kt * BN;
        const int ahead = ti + nstages - 1;
        if (ahead < ti_hi) fetch(ahead, (ahead - ti_lo) % nstages);
        else copies_commit();
        if (nstages == 2) copies_wait<1>();
        else if (nstages == 3) copies_wait<2>();
        else copies_wait<3>();
        __syncthreads();                                                  // tile ti has landed for every thread
        const __nv_bfloat16* Kt = Ks + ((ti - ti_lo) % nstages) * stage;
        const __nv_bfloat16* Vt = Vs + ((ti - ti_lo) % nstages) * stage;

        // a warp whose 16 rows lie beyond the tile's rows (a single token brings H/G rows) has nothing to compute
        if (rb * 16 < rows) {
            // S = Q K^T for this warp's 16 rows and the tile's 64 keys
            float sacc[BN / 8][4];
    #pragma unroll
            for (int i = 0; i < BN / 8; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
            for (int k0 = 0; k0 < D; k0 += 16) {
                uint32_t a[4];
                ldmatrix_x4(a, Qs + (rb * 16 + (lane & 15)) * DP + k0 + (lane >> 4) * 8);
    #pragma unroll
                for (int nt = 0; nt < BN / 8; nt += 2) {
                    uint32_t b[4];      // keys nt*8 .. nt*8+15: (b0, b1) of the first eight, (b0, b1) of the next eight
                    ldmatrix_x4(b, Kt + (nt * 8 + (lane & 7) + ((lane >> 4) << 3)) * DP + k0 + ((lane >> 3) & 1) * 8);
                    mma_bf16(sacc[nt], a, b[0], b[1]);
                    mma_bf16(sacc[nt + 1], a, b[2], b[3]);
                }
            }
            // scale, mask, and the tile's maximum per row.  A tile that every row of the CTA sees whole needs no mask.
            const bool whole = rows == BM && j0 + BN - 1 <= pos0 && (window <= 0 || pos_last - j0 < window || j0 + BN - 1 < keep_first);
            float tmax[2] = {-INFINITY, -INFINITY};
            if (whole) {
    #pragma unroll
                for (int nt = 0; nt < BN / 8; ++nt) {
    #pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        sacc[nt][e] *= sl2;
                        tmax[e >> 1] = fmaxf(tmax[e >> 1], sacc[nt][e]);
                    }
                }
            } else {
    #pragma unroll
                for (int nt = 0; nt < BN / 8; ++nt) {
    #pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = j0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                        const bool hi = e >= 2;
                        const bool ok = (hi ? live_hi : live_lo) && visible(hi ? pos_hi : pos_lo, j, window, keep_first);
                        const float s = ok ? sacc[nt][e] * sl2 : -INFINITY;
                        sacc[nt][e] = s;
                        tmax[hi] = fmaxf(tmax[hi], s);
                    }
                }
            }
            float alpha[2], base[2];
    #pragma unroll
            for (int h = 0; h < 2; ++h) {
                tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
                tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
                const float m_new = fmaxf(row_m[h], tmax[h]);
                base[h] = m_new == -INFINITY ? 0.f : m_new;                   // a row that has seen nothing yet
                alpha[h] = ex2(row_m[h] - base[h]);                         // exp2(-inf) = 0
                row_m[h] = m_new;
            }
            float tsum[2] = {0.f, 0.f};
            uint32_t pa[BN / 16][4];                                          // P as the A operand, 16 keys per k-step
    #pragma unroll
            for (int nt = 0; nt < BN / 8; ++nt) {
                const float p0 = ex2(sacc[nt][0] - base[0]), p1 = ex2(sacc[nt][1] - base[0]);
                const float p2 = ex2(sacc[nt][2] - base[1]), p3 = ex2(sacc[nt][3] - base[1]);
                tsum[0] += p0 + p1;
                tsum[1] += p2 + p3;
                pa[nt >> 1][(nt & 1) * 2] = pack_bf16(p0, p1);
                pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
    #pragma unroll
            for (int h = 0; h < 2; ++h) {
                tsum[h] += __shfl_xor_sync(0xffffffffu, tsum[h], 1);
                tsum[h] += __shfl_xor_sync(0xffffffffu, tsum[h], 2);
                row_l[h] = row_l[h] * alpha[h] + tsum[h];
            }
    #pragma unroll
            for (int i = 0; i < VC / 8; ++i) {
                if (i >= ntw) break;
                oacc[i][0] *= alpha[0];
                oacc[i][1] *= alpha[0];
                oacc[i][2] *= alpha[1];
                oacc[i][3] *= alpha[1];
            }
            // O += P V
    #pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
    #pragma unroll
                for (int nt = 0; nt < VC / 8; nt += 2) {
                    if (nt >= ntw) break;                                 // (the same for the whole warp)
                    uint32_t b[4];      // keys kk*16 .. +15 (rows), columns cb + nt*8 .. +15: matrices (k lo, n lo), (k hi, n lo), (k lo, n hi), (k hi, n hi)
                    ldmatrix_x4_trans(b, Vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VP + cb + nt * 8 + (lane >> 4) * 8);
                    mma_bf16(oacc[nt], pa[kk], b[0], b[1]);
                    mma_bf16(oacc[nt + 1], pa[kk], b[2], b[3]);
                }
            }
        }
        __syncthreads();                                                  // before a later fetch writes into this buffer
    }
    // normalise and store this chunk's columns of u (one run of tiles: final; several: as they are, beside maximum and sum)
    const float inv[2] = {nsplit > 1 ? 1.0f : (row_l[0] > 0.f ? 1.0f / row_l[0] : 0.f), nsplit > 1 ? 1.0f : (row_l[1] > 0.f ? 1.0f / row_l[1] : 0.f)};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = h ? r_hi : r_lo;
        if (r >= rows) continue;
        const size_t row_index = (size_t)(t0 + r / Gq) * H + c * Gq + r % Gq;
        float* dst = u + ((size_t)sp * T * H + row_index) * GE;
        if (nsplit > 1 && blockIdx.z == 0 && (lane & 3) == 0 && (!colsplit || warp == 0)) {
            part_ml[((size_t)sp * T * H + row_index) * 2] = row_m[h];
            part_ml[((size_t)sp * T * H + row_index) * 2 + 1] = row_l[h];
        }
#pragma unroll
        for (int nt = 0; nt < VC / 8; ++nt) {
            if (nt >= ntw) break;
            const int col = v0 + cb + nt * 8 + (lane & 3) * 2;
            if (col < GE) *reinterpret_cast<float2*>(dst + col) = make_float2(oacc[nt][2 * h] * inv[h], oacc[nt][2 * h + 1] * inv[h]);
        }
    }
}

// out[t, h, e] = gate[t, h] * sum_g mix[h, g] u[t, g, kv(h) * E + e]      (mix null: u[t, h, ...] alone)
// One CTA per (token, key/value head c): the H x E block of u that the query heads of c read goes to shared memory
// once (rows of E consecutive numbers), then a thread per (head of c, channel) takes its sum over g.
__global__ void __launch_bounds__(256)
headmix_combine_kernel(const float* __restrict__ u, const float* __restrict__ part_ml, int nsplit, int T, const float* __restrict__ mix,
                       const float* __restrict__ gate, __nv_bfloat16* __restrict__ out, int H, int G, int E) {
    extern __shared__ float sm[];
    forge::pdl_launch_dependents();
    const int t = blockIdx.x, c = blockIdx.y, GE = G * E, Gq = H / G;
    float* mx = sm;                     // [Gq][H] rows of mix of this group's heads
    float* ub = sm + (mix ? Gq * H : 0);     // [H][E]
    if (mix) for (int i = threadIdx.x; i < Gq * H; i += blockDim.x) mx[i] = mix[(size_t)c * Gq * H + i];
    forge::pdl_wait();
    const float* ut = u + (size_t)t * H * GE + (size_t)c * E;
    // Several runs of key tiles (nsplit > 1): run s of head g counts with 2^(m_s - m) / sum_s 2^(m_s - m) l_s; a thread per
    // head works the weights out once, then every value is nsplit independent loads.
    float* wsp = ub + (mix || nsplit > 1 ? H * E : 0);     // [H][nsplit]
    if (nsplit > 1) {
        for (int g = threadIdx.x; g < H; g += blockDim.x) {
            float m = -INFINITY, den = 0.f;
            for (int sp = 0; sp < nsplit; ++sp) m = fmaxf(m, part_ml[((size_t)sp * T * H + (size_t)t * H + g) * 2]);
            for (int sp = 0; sp < nsplit; ++sp) {
                const size_t row = (size_t)sp * T * H + (size_t)t * H + g;
                const float l = part_ml[row * 2 + 1];
                const float w = l > 0.f ? exp2f(part_ml[row * 2] - m) : 0.f;        // a run that saw no key counts for nothing
                wsp[g * nsplit + sp] = w;
                den = fmaf(w, l, den);
            }
            const float inv = den > 0.f ? 1.0f / den : 0.f;
            for (int sp = 0; sp < nsplit; ++sp) wsp[g * nsplit + sp] *= inv;
        }
        __syncthreads();
    }
    auto u_of = [&](int g, int e) {
        if (nsplit <= 1) return ut[(size_t)g * GE + e];
        float a = 0.f;
        for (int sp = 0; sp < nsplit; ++sp) {
            const float w = wsp[g * nsplit + sp];
            if (w > 0.f) a = fmaf(w, u[((size_t)sp * T * H + (size_t)t * H + g) * GE + (size_t)c * E + e], a);
        }
        return a;
    };
    if (mix || nsplit > 1) {
        for (int i = threadIdx.x; i < H * E; i += blockDim.x) ub[i] = u_of(i / E, i % E);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < Gq * E; i += blockDim.x) {
        const int hq = i / E, e = i % E, h = c * Gq + hq;
        float a;
        if (mix) {
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            int g = 0;
            for (; g + 3 < H; g += 4) {
                a0 = fmaf(mx[hq * H + g], ub[g * E + e], a0);
                a1 = fmaf(mx[hq * H + g + 1], ub[(g + 1) * E + e], a1);
                a2 = fmaf(mx[hq * H + g + 2], ub[(g + 2) * E + e], a2);
                a3 = fmaf(mx[hq * H + g + 3], ub[(g + 3) * E + e], a3);
            }
            for (; g < H; ++g) a0 = fmaf(mx[hq * H + g], ub[g * E + e], a0);
            a = (a0 + a1) + (a2 + a3);
        } else {
            a = nsplit > 1 ? ub[h * E + e] : ut[(size_t)h * GE + e];
        }
        if (gate) a *= gate[(size_t)t * H + h];
        out[((size_t)t * H + h) * E + e] = __float2bfloat16_rn(a);
    }
}

forge::PerDeviceFlag g_attr_done[3], g_combine_done;

template <int VC>
int launch_mma(int which, dim3 grid, size_t smem, cudaStream_t stream, const __nv_bfloat16* q, const __nv_bfloat16* cache,
               const int32_t* bt, const int32_t* tok_req, const int32_t* positions, const int32_t* t0, const int32_t* tn, float* u,
               float* part_ml, int nsplit, int nstages, int qrows, int T, int H, int G, int D, int E, int page_size, long long page_stride,
               int max_pages, int window, int keep_first, float scale) {
    bool& done = g_attr_done[which].current();
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(headmix_mma_kernel<VC>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMmaSmemLimit);
        if (e != cudaSuccess) return forge::check_launch("headmix_attention_mma (shared memory)", e);
        done = true;
    }
    return forge::check_launch("headmix_attention_mma",
                               forge::launch(headmix_mma_kernel<VC>, grid, dim3(kThreads), smem, stream, 1, q, cache, bt, tok_req, positions,
                                             t0, tn, u, part_ml, nsplit, nstages, qrows, T, H, G, D, E, page_size, page_stride, max_pages, window, keep_first, scale));
}

}  // namespace

// 1 if the tensor-core kernels take these sizes: key heads of a multiple of 16 channels up to 128, value heads of a
// multiple of 8 channels, at most 64 query heads per key/value head, at most 96 heads (the exchange matrix in shared memory),
// pages of a power of two tokens.
extern "C" int forge_headmix_mma_supports(int H, int G, int D, int E, int page_size) {
    return (page_size > 0 && (page_size & (page_size - 1)) == 0 && H > 0 && G > 0 && H % G == 0 && H / G <= BM && H <= 96 && D % 16 == 0 && D >= 16 && D <= 128 && E % 8 == 0 && E > 0) ? 1 : 0;
}

// q bf16 [T, H*D]; u fp32 [nsplit, T, H, G*E] (scratch); part_ml fp32 [nsplit, T, H, 2] (scratch, nsplit > 1: steps of single
// tokens whose key tiles are dealt out to nsplit CTAs); out bf16 [T, H*E].  tile_t0 / tile_n: tiles of consecutive tokens of one
// request with tile_n * (H/G) <= 64 (both null: one token per tile, num_tiles = T).  mix fp32 [H, H] or null; gate fp32
// [T, H] or null.
extern "C" int forge_headmix_attention_mma(const void* q, const void* cache, const int32_t* block_table, const int32_t* tok_req,
                                           const int32_t* positions, const int32_t* tile_t0, const int32_t* tile_n, const float* mix,
                                           const float* gate, float* u, float* part_ml, int nsplit, void* out, int T, int num_tiles, int H, int G, int D, int E,
                                           int page_size, long long page_stride, int max_pages, int window, int keep_first, float scale,
                                           cudaStream_t stream) {
    if (!forge_headmix_mma_supports(H, G, D, E, page_size)) return forge::fail(FORGE_ERR_UNSUPPORTED, "headmix_attention_mma: H=%d G=%d D=%d E=%d", H, G, D, E);
    if (T < 0 || num_tiles < 0 || page_size <= 0 || max_pages <= 0 || keep_first < 0 || (tile_t0 == nullptr) != (tile_n == nullptr))
        return forge::fail(FORGE_ERR_ARG, "headmix_attention_mma: bad arguments");
    if (T == 0 || num_tiles == 0) return FORGE_OK;
    if (nsplit < 1 || nsplit > 16 || (nsplit > 1 && (tile_t0 != nullptr || part_ml == nullptr)))
        return forge::fail(FORGE_ERR_ARG, "headmix_attention_mma: the keys are dealt out to several CTAs only in steps of single tokens");
    const int GE = G * E;
    int VC = 64;                        // the chunk width that wastes the fewest columns; among equals the widest
    for (int cand : {128, 256})
        if ((GE + cand - 1) / cand * cand <= (GE + VC - 1) / VC * VC) VC = cand;
    const int chunks = (GE + VC - 1) / VC;
    // buffers for key/value tiles: two.  (Three and four for steps of single tokens measured no faster at 8 requests and
    // slower at 64, where they cost the second CTA of an SM: such a step's time is the live warps' tensor work, not the copies.)
    // a step of single tokens brings H/G rows a tile: 16 rows of queries in shared memory leave room for a second CTA on the SM
    const int qrows = (tile_t0 == nullptr && H / G <= 16) ? 16 : BM;
    const size_t q_bytes = sizeof(__nv_bfloat16) * (size_t)qrows * (D + kPad);
    const size_t stage_bytes = sizeof(__nv_bfloat16) * (size_t)BN * ((D + kPad) + (VC + kPad));
    const int nstages = 2;
    const size_t smem = q_bytes + nstages * stage_bytes;
    const dim3 grid(num_tiles * nsplit, G, chunks);
    const __nv_bfloat16* qb = (const __nv_bfloat16*)q;
    const __nv_bfloat16* cb = (const __nv_bfloat16*)cache;
    int rc;
    if (VC == 64) rc = launch_mma<64>(0, grid, smem, stream, qb, cb, block_table, tok_req, positions, tile_t0, tile_n, u, part_ml, nsplit, nstages, qrows, T, H, G, D, E, page_size, page_stride, max_pages, window, keep_first, scale);
    else if (VC == 128) rc = launch_mma<128>(1, grid, smem, stream, qb, cb, block_table, tok_req, positions, tile_t0, tile_n, u, part_ml, nsplit, nstages, qrows, T, H, G, D, E, page_size, page_stride, max_pages, window, keep_first, scale);
    else rc = launch_mma<256>(2, grid, smem, stream, qb, cb, block_table, tok_req, positions, tile_t0, tile_n, u, part_ml, nsplit, nstages, qrows, T, H, G, D, E, page_size, page_stride, max_pages, window, keep_first, scale);
    if (rc != FORGE_OK) return rc;
    const size_t csmem = sizeof(float) * ((mix ? (size_t)(H / G) * H : 0) + (mix || nsplit > 1 ? (size_t)H * E : 0) + (nsplit > 1 ? (size_t)H * nsplit : 0));
    if (csmem > 160 * 1024) return forge::fail(FORGE_ERR_UNSUPPORTED, "headmix_combine: %d heads of %d channels", H, E);
    bool& cdone = g_combine_done.current();
    if (!cdone) {
        cudaError_t e = cudaFuncSetAttribute(headmix_combine_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        if (e != cudaSuccess) return forge::check_launch("headmix_combine (shared memory)", e);
        cdone = true;
    }
    return forge::check_launch("headmix_combine", forge::launch(headmix_combine_kernel, dim3(T, G), dim3(256), csmem, stream, 1,
                                                                (const float*)u, (const float*)part_ml, nsplit, T, mix, gate, (__nv_bfloat16*)out, H, G, E));
}

FORGE_DEFINE_CHECKS_ENTRY(attention_headmix_mma)
