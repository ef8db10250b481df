// Operators of mixers that carry a matrix per request and head from token to token, of gated heads, and of the
// hashed pair embedding.
//
//   matrix_state_scan   S_t = decay_t S_{t-1} + gain_t k_t v_t^T, o_t = S_t^T q_t over the tokens of every segment, from
//                       and into the request's state slot; two forms of decay (below)
//   head_norm_gate      out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w * act(gate[t, h, :]) * scale
//   head_gate           out[t, h, :] = x[t, h, :] * sigmoid(gate[t, h]) * scale
//   bigram_embed        h[r] += table[(previous token * a + token * b) mod buckets], the table's last row at position 0;
//                       then the request's previous token becomes the last one of its segment
//
// The scan keeps everything in float32.  A warp owns CPW value channels (columns of S) of one head; lane l holds the
// key channels l, l + 32, ... of those columns in registers for the whole segment, so a token costs two fused
// multiply-adds per held number and one shuffle tree per column; the rows of 32 tokens at a time are staged in shared
// memory by the whole block, and the exponential gates of those tokens are computed once for the block.  A column's sum over the key channels
// is taken in one order (lane-local over l + 32 i, then the xor tree), whatever the step holds: a token's result is
// bit for bit the same in a prompt, a portion or alone.  State layout: [slot, head, value channel, key channel].
//
// Long segments are cut into chunks of L tokens that run side by side, in three launches: (1) every chunk but a
// segment's last is scanned from an empty state and leaves its end state and its total decay in scratch; (2) per
// segment, the chunks' start states follow one from the other (start[c + 1] = decay[c] start[c] + local[c], for the
// exponential gates with their maxima: m' = max(F + m, m_local), weights e^{F + m - m'} and e^{m_local - m'}); (3) every
// chunk is scanned again from its start state, now with read-outs, and a segment's last chunk leaves the state in the
// slot.  The arithmetic per token is the same as in one piece; the start states differ from it by float32 rounding.
#include "common.cuh"

enum { SCAN_CHANNEL_DECAY = 0, SCAN_EXP_GATES = 1 };

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// SCAN_CHANNEL_DECAY: decay per key channel d = sigmoid(z[r, h, d])^(1 / p0), gain 1; the launcher turns the logits z
//                     (`gate`, row stride gate_stride) into the decays in place before the scan, once for all warps.
// SCAN_EXP_GATES:     per head i = p0 tanh(gate[r, g0 + h] / p0), f = logsigmoid(p0 tanh(gate[r, g1 + h] / p0));
//                     m' = max(f + m, i); decay e^{f + m - m'}, gain e^{i - m'}; n' = decay n + gain k;
//                     o = S'^T q / (max(|n' . q|, e^{-m'}) + floor).  n: [slot, head, key channel], m: [slot, head].
// grid (column blocks, heads, segments); the exponential-gate form takes one block per head (its n and m are read by
// every warp at the start and written by the first at the end, with a barrier in between).
// Scratch of the chunked form; chunk ids count the chunks of all segments in the order of the segments.
struct ScanChunks {
    int L, S;              // tokens in a chunk; segments in the step
    float* local_S;        // [chunk, H, Dv, D]   end state of the chunk scanned from an empty state
    float* local_vec;      // [chunk, H, D]       channel decay: the product of the chunk's decays; exponential gates: its normaliser
    float* local_F;        // [chunk, H]          exponential gates: the sum of the chunk's log forget gates
    float* local_m;        // [chunk, H]          exponential gates: the chunk's maximum from an empty state
    float* start_S;        // [chunk, H, Dv, D]   state before the chunk's first token
    float* start_vec;      // [chunk, H, D]       exponential gates: the normaliser there
    float* start_m;        // [chunk, H]          exponential gates: the maximum there
};

// Which (segment, chunk of it) the chunk id is; false beyond the step's last chunk.
__device__ __forceinline__ bool find_chunk(int id, const ScanChunks& ch, const int* seg_q_len, int& seg, int& index, int& count,
                                           int& first_id) {
    int at = 0;
    for (int s = 0; s < ch.S; ++s) {
        const int nc = (seg_q_len[s] + ch.L - 1) / ch.L;
        if (id < at + nc) {
            seg = s; index = id - at; count = nc; first_id = at;
            return true;
        }
        at += nc;
    }
    return false;
}

enum { SCAN_WHOLE = 0, SCAN_LOCAL = 1, SCAN_FROM_START = 3 };

// PASS: SCAN_WHOLE - grid z counts segments, from and into the slots.  SCAN_LOCAL / SCAN_FROM_START - grid z counts
// chunks (launches (1) and (3) of the chunked form).
template <int MODE, int RPL, int CPW, int PASS>
__global__ void __launch_bounds__(MODE == SCAN_EXP_GATES ? 1024 : 256) matrix_state_scan_kernel(
    const float* __restrict__ proj, int P, int q_col, int k_col, int v_col, const float* __restrict__ gate, int gate_stride,
    int g0, int g1, float p0, float q_scale, float floor_, const int* __restrict__ seg_q_start,
    const int* __restrict__ seg_q_len, const int* __restrict__ seg_slot, float* __restrict__ memory,
    float* __restrict__ normalizer, float* __restrict__ maximum, float* __restrict__ out, int H, int D, int Dv, ScanChunks ch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int h = blockIdx.y;
    const int c0 = (blockIdx.x * warps + warp) * CPW;
    int seg = blockIdx.z, chunk = 0, chunks = 1, first_id = 0;
    if (PASS != SCAN_WHOLE && !find_chunk(blockIdx.z, ch, seg_q_len, seg, chunk, chunks, first_id)) return;
    const bool last_chunk = chunk == chunks - 1;
    if (PASS == SCAN_LOCAL && last_chunk) return;              // nobody starts from its end
    int r0 = seg_q_start[seg], n_rows = seg_q_len[seg];
    const int slot = seg_slot[seg];
    if (PASS != SCAN_WHOLE) {
        r0 += chunk * ch.L;
        n_rows = min(ch.L, n_rows - chunk * ch.L);
    }
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float gate_s[3][32], max_s[33], carry_s[2];     // exponential gates: see the loop
    float S[CPW][RPL], nz[RPL], total[RPL], m = 0.f;
    float* mem = memory + ((size_t)slot * H + h) * Dv * D;
    const size_t cid = (size_t)blockIdx.z * H + h;             // (chunk id, head) in the scratch arrays
    const float* from = PASS == SCAN_FROM_START ? ch.start_S + cid * Dv * D : mem;
#pragma unroll
    for (int c = 0; c < CPW; ++c)
#pragma unroll
        for (int i = 0; i < RPL; ++i) {
            const int d = lane + 32 * i;
            S[c][i] = (PASS != SCAN_LOCAL && c0 + c < Dv && d < D) ? from[(size_t)(c0 + c) * D + d] : 0.f;
        }
#pragma unroll
    for (int i = 0; i < RPL; ++i) total[i] = 1.f;
    if (MODE == SCAN_EXP_GATES) {
        const float* n_from = PASS == SCAN_FROM_START ? ch.start_vec + cid * D : normalizer + ((size_t)slot * H + h) * D;
#pragma unroll
        for (int i = 0; i < RPL; ++i) {
            const int d = lane + 32 * i;
            nz[i] = (PASS != SCAN_LOCAL && d < D) ? n_from[d] : 0.f;
        }
        m = PASS == SCAN_LOCAL ? -FLT_MAX : PASS == SCAN_FROM_START ? ch.start_m[cid] : maximum[(size_t)slot * H + h];
        if (threadIdx.x == 0) {
            carry_s[0] = m;                        // the running maximum, and the sum of the log forget gates
            carry_s[1] = 0.f;
        }
        // Every warp has read n and m before the first may write them (the loop's first barrier comes before any write).
    }
    // The rows of 32 tokens at a time are staged in shared memory by the whole block (one round of loads in flight
    // instead of one per token): q and k of the head, the decays (channel-decay form), and the block's value channels.
    extern __shared__ float tile_s[];
    const int VC = warps * CPW, v_base = blockIdx.x * VC;
    float* q_s = tile_s;                                       // [32][D]
    float* k_s = q_s + 32 * D;                                 // [32][D]
    float* a_s = k_s + 32 * D;                                 // [32][D], channel-decay form only
    float* v_s = a_s + (MODE == SCAN_CHANNEL_DECAY ? 32 * D : 0);   // [32][VC]
    for (int t = 0; t < n_rows; ++t) {
        const int r = r0 + t, tt = t & 31;
        if (tt == 0) {
            __syncthreads();                                   // the tile before has been used up
            const int rows = min(32, n_rows - t);
            for (int idx = threadIdx.x; idx < rows * D; idx += blockDim.x) {
                const int row = idx / D, d = idx - row * D;
                const float* src = proj + (size_t)(r + row) * P;
                q_s[idx] = src[q_col + h * D + d];
                k_s[idx] = src[k_col + h * D + d];
                if (MODE == SCAN_CHANNEL_DECAY) a_s[idx] = gate[(size_t)(r + row) * gate_stride + g0 + h * D + d];
            }
            for (int idx = threadIdx.x; idx < rows * VC; idx += blockDim.x) {
                const int row = idx / VC, c = idx - row * VC;
                v_s[idx] = v_base + c < Dv ? proj[(size_t)(r + row) * P + v_col + h * Dv + v_base + c] : 0.f;
            }
            if (MODE == SCAN_CHANNEL_DECAY) __syncthreads();
            if (MODE == SCAN_EXP_GATES) {
                // The gates of the tile's tokens, once for the block: thread j takes token t + j's two logarithms, the
                // first thread walks the maximum through them, then thread j takes the token's three exponentials.
                const int j = threadIdx.x;
                float li = 0.f, lf = 0.f;
                if (j < 32 && t + j < n_rows) {
                    const float* grow = gate + (size_t)(r + j) * gate_stride;
                    li = p0 * tanhf(grow[g0 + h] / p0);
                    lf = log_sigmoid(p0 * tanhf(grow[g1 + h] / p0));
                    gate_s[0][j] = lf;
                    gate_s[1][j] = li;
                }
                __syncthreads();
                if (j == 0) {
                    float mm = carry_s[0], ff = carry_s[1];
                    for (int u = 0; u < 32 && t + u < n_rows; ++u) {
                        max_s[u] = mm;                               // the maximum before token t + u
                        mm = fmaxf(gate_s[0][u] + mm, gate_s[1][u]);
                        ff += gate_s[0][u];
                    }
                    max_s[32] = mm;
                    carry_s[1] = ff;
                }
                __syncthreads();
                if (j < 32 && t + j < n_rows) {
                    const float before = max_s[j], after = fmaxf(lf + before, li);
                    gate_s[0][j] = expf(lf + before - after);
                    gate_s[1][j] = expf(li - after);
                    gate_s[2][j] = expf(-after);
                }
                if (j == 0) carry_s[0] = max_s[32];
                __syncthreads();
            }
        }
        float qc[RPL], kc[RPL], ac[RPL], vc[CPW];
#pragma unroll
        for (int i = 0; i < RPL; ++i) {
            const int d = lane + 32 * i;
            qc[i] = d < D ? q_s[tt * D + d] * q_scale : 0.f;
            kc[i] = d < D ? k_s[tt * D + d] : 0.f;
            ac[i] = (MODE == SCAN_CHANNEL_DECAY && d < D) ? a_s[tt * D + d] : 0.f;
        }
#pragma unroll
        for (int c = 0; c < CPW; ++c) vc[c] = v_s[tt * VC + warp * CPW + c];
        float keep = 1.f, take = 1.f, denom = 1.f;
        if (MODE == SCAN_EXP_GATES) {
            keep = gate_s[0][tt];
            take = gate_s[1][tt];
            float part = 0.f;
#pragma unroll
            for (int i = 0; i < RPL; ++i) {
                nz[i] = keep * nz[i] + take * kc[i];
                part += nz[i] * qc[i];
            }
            if (PASS != SCAN_LOCAL) denom = 1.f / (fmaxf(fabsf(warp_sum(part)), gate_s[2][tt]) + floor_);
        } else if (PASS == SCAN_LOCAL) {
#pragma unroll
            for (int i = 0; i < RPL; ++i) total[i] *= ac[i];
        }
        if (PASS == SCAN_LOCAL) {                 // the state only
#pragma unroll
            for (int c = 0; c < CPW; ++c)
#pragma unroll
                for (int i = 0; i < RPL; ++i) {
                    if (MODE == SCAN_CHANNEL_DECAY) S[c][i] = ac[i] * S[c][i] + kc[i] * vc[c];
                    else S[c][i] = keep * S[c][i] + take * (kc[i] * vc[c]);
                }
            continue;
        }
        float o[CPW];
#pragma unroll
        for (int c = 0; c < CPW; ++c) {
            float part = 0.f;
#pragma unroll
            for (int i = 0; i < RPL; ++i) {
                if (MODE == SCAN_CHANNEL_DECAY) S[c][i] = ac[i] * S[c][i] + kc[i] * vc[c];
                else S[c][i] = keep * S[c][i] + take * (kc[i] * vc[c]);
                part += S[c][i] * qc[i];
            }
            o[c] = warp_sum(part);
            if (MODE == SCAN_EXP_GATES) o[c] = o[c] * denom;
        }
#pragma unroll
        for (int c = 0; c < CPW; ++c)
            if (lane == c && c0 + c < Dv) out[(size_t)r * H * Dv + h * Dv + c0 + c] = o[c];
    }
    if (n_rows <= 0) return;
    if (PASS == SCAN_FROM_START && !last_chunk) return;        // only a segment's last chunk leaves the state in the slot
    float* to = PASS == SCAN_LOCAL ? ch.local_S + cid * Dv * D : mem;
#pragma unroll
    for (int c = 0; c < CPW; ++c)
#pragma unroll
        for (int i = 0; i < RPL; ++i) {
            const int d = lane + 32 * i;
            if (c0 + c < Dv && d < D) to[(size_t)(c0 + c) * D + d] = S[c][i];
        }
    if (blockIdx.x != 0 || warp != 0) return;
    if (MODE == SCAN_CHANNEL_DECAY) {
        if (PASS == SCAN_LOCAL)
#pragma unroll
            for (int i = 0; i < RPL; ++i) {
                const int d = lane + 32 * i;
                if (d < D) ch.local_vec[cid * D + d] = total[i];
            }
        return;
    }
    float* n_to = PASS == SCAN_LOCAL ? ch.local_vec + cid * D : normalizer + ((size_t)slot * H + h) * D;
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
        const int d = lane + 32 * i;
        if (d < D) n_to[d] = nz[i];
    }
    if (lane == 0) {                                           // thread 0: it wrote the carries itself
        if (PASS == SCAN_LOCAL) {
            ch.local_m[cid] = carry_s[0];
            ch.local_F[cid] = carry_s[1];
        } else {
            maximum[(size_t)slot * H + h] = carry_s[0];
        }
    }
}

// z -> sigmoid(z)^(1 / tau) = exp(logsigmoid(z) / tau), in place.
__global__ void channel_decay_kernel(float* __restrict__ z, size_t total, float tau) {
    pdl_wait();
    pdl_launch_dependents();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        z[i] = expf(log_sigmoid(z[i]) / tau);
}

// Launch (2) of the chunked form: one block per (head, segment) walks the segment's chunks in order.
template <int MODE>
__global__ void scan_chunk_starts_kernel(const int* __restrict__ seg_q_len, const int* __restrict__ seg_slot,
                                         const float* __restrict__ memory, const float* __restrict__ normalizer,
                                         const float* __restrict__ maximum, int H, int D, int Dv, ScanChunks ch) {
    pdl_wait();
    pdl_launch_dependents();
    const int h = blockIdx.x, seg = blockIdx.y;
    int first = 0;
    for (int s = 0; s < seg; ++s) first += (seg_q_len[s] + ch.L - 1) / ch.L;
    const int chunks = (seg_q_len[seg] + ch.L - 1) / ch.L;
    if (chunks <= 0) return;
    const int slot = seg_slot[seg];
    const size_t per = (size_t)Dv * D;
    const float* mem = memory + ((size_t)slot * H + h) * per;
    for (size_t e = threadIdx.x; e < per; e += blockDim.x) {
        const int d = (int)(e % D);
        float s = mem[e];
        float m = MODE == SCAN_EXP_GATES ? maximum[(size_t)slot * H + h] : 0.f;
        for (int c = 0; c < chunks; ++c) {
            const size_t cid = (size_t)(first + c) * H + h;
            ch.start_S[cid * per + e] = s;
            if (c + 1 == chunks) break;
            if (MODE == SCAN_CHANNEL_DECAY) {
                s = ch.local_vec[cid * D + d] * s + ch.local_S[cid * per + e];
            } else {
                const float F = ch.local_F[cid], ml = ch.local_m[cid];
                const float m1 = fmaxf(F + m, ml);
                s = expf(F + m - m1) * s + expf(ml - m1) * ch.local_S[cid * per + e];
                m = m1;
            }
        }
    }
    if (MODE == SCAN_EXP_GATES)
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            float n = normalizer[((size_t)slot * H + h) * D + d];
            float m = maximum[(size_t)slot * H + h];
            for (int c = 0; c < chunks; ++c) {
                const size_t cid = (size_t)(first + c) * H + h;
                ch.start_vec[cid * D + d] = n;
                if (d == 0) ch.start_m[cid] = m;
                if (c + 1 == chunks) break;
                const float F = ch.local_F[cid], ml = ch.local_m[cid];
                const float m1 = fmaxf(F + m, ml);
                n = expf(F + m - m1) * n + expf(ml - m1) * ch.local_vec[cid * D + d];
                m = m1;
            }
        }
}

template <int MODE, int RPL, int CPW>
static void launch_scan(const float* proj, int P, int q_col, int k_col, int v_col, const float* gate, int gate_stride, int g0, int g1,
                        float p0, float q_scale, float floor_, const int* seg_q_start, const int* seg_q_len, const int* seg_slot,
                        float* memory, float* normalizer, float* maximum, float* out, int S, int H, int D, int Dv, ScanChunks ch,
                        int max_chunks, cudaStream_t stream) {
    const int total_warps = (Dv + CPW - 1) / CPW;
    // The exponential-gate form: all of a head's columns in one block.  The other: blocks of up to 8 warps.
    const int warps = MODE == SCAN_EXP_GATES ? total_warps : (total_warps < 8 ? total_warps : 8);
    const int col_blocks = (total_warps + warps - 1) / warps;
    const size_t smem = (size_t)32 * ((MODE == SCAN_CHANNEL_DECAY ? 3 : 2) * D + warps * CPW) * sizeof(float);
#define KVB_SCAN_PASS(PASS, Z)                                                                                                  \
    do {                                                                                                                        \
        if (smem + 2048 > 48 * 1024)                                                                                            \
            cudaFuncSetAttribute(matrix_state_scan_kernel<MODE, RPL, CPW, PASS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        kvb_launch(matrix_state_scan_kernel<MODE, RPL, CPW, PASS>, dim3(col_blocks, H, Z), dim3(32 * warps), smem, stream, proj, P,  \
                   q_col, k_col, v_col, gate, gate_stride, g0, g1, p0, q_scale, floor_, seg_q_start, seg_q_len, seg_slot, memory,    \
                   normalizer, maximum, out, H, D, Dv, ch);                                                                     \
    } while (0)
    if (max_chunks <= 0) {
        KVB_SCAN_PASS(SCAN_WHOLE, S);
        return;
    }
    KVB_SCAN_PASS(SCAN_LOCAL, max_chunks);
    kvb_launch(scan_chunk_starts_kernel<MODE>, dim3(H, S), dim3(256), 0, stream, seg_q_len, seg_slot, (const float*)memory,
               (const float*)normalizer, (const float*)maximum, H, D, Dv, ch);
    KVB_SCAN_PASS(SCAN_FROM_START, max_chunks);
#undef KVB_SCAN_PASS
}

// proj: float32 [T, P] with q at q_col (H * D numbers), k at k_col, v at v_col (H * Dv).  `gate`: float32 rows of
// stride gate_stride - per-channel decay logits [T, H * D] (mode 0; overwritten by the decays), or the two gates'
// pre-activations at g0 and g1 (mode 1).
// `max_chunks` > 0: the chunked form with chunks of `chunk_len` tokens; `max_chunks` bounds the step's chunk count
// (sum over segments of ceil(len / chunk_len)) and `scratch` holds that many times H * (2 Dv D + 2 D + 3) floats.
// scratch floats: max_chunks * H * (2 * Dv * D + 2 * D + 3).

KVB_API int kvb_matrix_state_scan(int mode, const float* proj, int P, int q_col, int k_col, int v_col, const float* gate,
                                  int gate_stride, int g0, int g1, float p0, float q_scale, float floor_, const int* seg_q_start,
                                  const int* seg_q_len, const int* seg_slot, float* memory, float* normalizer, float* maximum,
                                  float* out, int T, int S, int H, int D, int Dv, int chunk_len, int max_chunks, float* scratch,
                                  cudaStream_t stream) {
    if (S <= 0) return KVB_OK;
    if (H < 1 || D < 1 || Dv < 1 || (mode != SCAN_CHANNEL_DECAY && mode != SCAN_EXP_GATES)) return KVB_ERR_SHAPE;
    if (D > 256 || Dv > 256 || H > 65535 || S > 65535 || max_chunks > 65535) return KVB_ERR_LIMIT;
    if (max_chunks > 0 && (chunk_len < 1 || scratch == nullptr)) return KVB_ERR_SHAPE;
    ScanChunks ch = {};
    if (max_chunks > 0) {
        const size_t states = (size_t)max_chunks * H * Dv * D, vecs = (size_t)max_chunks * H * D, ones = (size_t)max_chunks * H;
        ch.L = chunk_len;
        ch.S = S;
        ch.local_S = scratch;
        ch.start_S = ch.local_S + states;
        ch.local_vec = ch.start_S + states;
        ch.start_vec = ch.local_vec + vecs;
        ch.local_F = ch.start_vec + vecs;
        ch.local_m = ch.local_F + ones;
        ch.start_m = ch.local_m + ones;
    }
    if (mode == SCAN_CHANNEL_DECAY) {
        if (g0 != 0 || gate_stride != H * D) return KVB_ERR_SHAPE;       // the logits are rows of their own
        const size_t total = (size_t)T * H * D;
        size_t blocks = (total + 255) / 256;
        const size_t most = (size_t)kvb_sm_count() * 16;
        if (blocks > most) blocks = most;
        kvb_launch(channel_decay_kernel, dim3((int)blocks), dim3(256), 0, stream, const_cast<float*>(gate), total, p0);
    }
    const int rpl = D <= 32 ? 1 : D <= 64 ? 2 : D <= 128 ? 4 : 8;
    const int cpw = Dv <= 32 ? 1 : Dv <= 128 ? 4 : 8;
#define KVB_SCAN(MODE, RPL, CPW)                                                                                              \
    launch_scan<MODE, RPL, CPW>(proj, P, q_col, k_col, v_col, gate, gate_stride, g0, g1, p0, q_scale, floor_, seg_q_start,     \
                                seg_q_len, seg_slot, memory, normalizer, maximum, out, S, H, D, Dv, ch, max_chunks, stream)
#define KVB_SCAN_CPW(MODE, RPL)                                                                                               \
    do {                                                                                                                      \
        if (cpw == 1) KVB_SCAN(MODE, RPL, 1); else if (cpw == 4) KVB_SCAN(MODE, RPL, 4); else KVB_SCAN(MODE, RPL, 8);         \
    } while (0)
#define KVB_SCAN_RPL(MODE)                                                                                                    \
    do {                                                                                                                      \
        if (rpl == 1) KVB_SCAN_CPW(MODE, 1); else if (rpl == 2) KVB_SCAN_CPW(MODE, 2);                                        \
        else if (rpl == 4) KVB_SCAN_CPW(MODE, 4); else KVB_SCAN_CPW(MODE, 8);                                                 \
    } while (0)
    if (mode == SCAN_CHANNEL_DECAY) KVB_SCAN_RPL(SCAN_CHANNEL_DECAY); else KVB_SCAN_RPL(SCAN_EXP_GATES);
#undef KVB_SCAN_RPL
#undef KVB_SCAN_CPW
#undef KVB_SCAN
    return kvb_launch_status();
}

// ---------------------------------------------------------------------------------------------------------------
// One warp per (row, head).  o: float32 [T, H * Dv]; w: [Dv] (shared by the heads) or [H * Dv] (w_per_head);
// gate: float32 rows of stride gate_stride, the head's Dv numbers at gate_col + h * Dv; act 0: silu, 1: sigmoid.
// out (type T) rows of stride out_stride, written at out_col + h * Dv.
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, int w_per_head, float eps,
                                      const float* __restrict__ gate, int gate_stride, int gate_col, int act, float scale,
                                      T* __restrict__ out, int out_stride, int out_col, int pairs, int H, int Dv) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= pairs) return;
    const int t = pair / H, h = pair - t * H;
    const float* src = o + (size_t)t * H * Dv + (size_t)h * Dv;
    float ss = 0.f;
    for (int d = lane; d < Dv; d += 32) ss += src[d] * src[d];
    const float inv = 1.f / sqrtf(warp_sum(ss) / (float)Dv + eps);
    const float* g = gate + (size_t)t * gate_stride + gate_col + h * Dv;
    const float* wh = w + (w_per_head ? h * Dv : 0);
    T* dst = out + (size_t)t * out_stride + out_col + h * Dv;
    for (int d = lane; d < Dv; d += 32) {
        const float z = g[d];
        const float s = 1.f / (1.f + expf(-z));
        dst[d] = from_f32<T>(src[d] * inv * wh[d] * (act == 0 ? z * s : s) * scale);
    }
}

KVB_API int kvb_head_norm_gate(int out_dtype, const float* o, const float* w, int w_per_head, float eps, const float* gate,
                               int gate_stride, int gate_col, int act, float scale, void* out, int out_stride, int out_col,
                               int T, int H, int Dv, cudaStream_t stream) {
    if (T <= 0) return KVB_OK;
    if (H < 1 || Dv < 1 || act < 0 || act > 1) return KVB_ERR_SHAPE;
    const int pairs = T * H, warps = 4;
    dim3 grid((pairs + warps - 1) / warps), block(32 * warps);
    if (out_dtype == KVB_F32)
        kvb_launch(head_norm_gate_kernel<float>, grid, block, 0, stream, o, w, w_per_head, eps, gate, gate_stride, gate_col, act, scale,
                   (float*)out, out_stride, out_col, pairs, H, Dv);
    else if (out_dtype == KVB_BF16)
        kvb_launch(head_norm_gate_kernel<bf16>, grid, block, 0, stream, o, w, w_per_head, eps, gate, gate_stride, gate_col, act, scale,
                   (bf16*)out, out_stride, out_col, pairs, H, Dv);
    else
        return KVB_ERR_DTYPE;
    return kvb_launch_status();
}

// out[t, out_col + h * Dv + d] = x[t, h * Dv + d] * sigmoid(gate[t, gate_col + h]) * scale (gate null: no sigmoid).
template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ x, const T* __restrict__ gate, int gate_stride, int gate_col, float scale,
                                 T* __restrict__ out, int out_stride, int out_col, int H, int Dv, size_t total) {
    pdl_wait();
    pdl_launch_dependents();
    const int width = H * Dv;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / width;
        const int c = (int)(idx - t * width);
        float v = to_f32<T>(x[idx]) * scale;
        if (gate) v *= 1.f / (1.f + expf(-to_f32<T>(gate[t * gate_stride + gate_col + c / Dv])));
        out[t * out_stride + out_col + c] = from_f32<T>(v);
    }
}

KVB_API int kvb_head_gate(int dtype, const void* x, const void* gate, int gate_stride, int gate_col, float scale, void* out,
                          int out_stride, int out_col, int T, int H, int Dv, cudaStream_t stream) {
    const size_t total = (size_t)T * H * Dv;
    if (total == 0) return KVB_OK;
    size_t blocks = (total + 255) / 256;
    const size_t most = (size_t)kvb_sm_count() * 16;
    if (blocks > most) blocks = most;
    if (dtype == KVB_F32)
        kvb_launch(head_gate_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, (const float*)x, (const float*)gate, gate_stride,
                   gate_col, scale, (float*)out, out_stride, out_col, H, Dv, total);
    else if (dtype == KVB_BF16)
        kvb_launch(head_gate_kernel<bf16>, dim3((int)blocks), dim3(256), 0, stream, (const bf16*)x, (const bf16*)gate, gate_stride,
                   gate_col, scale, (bf16*)out, out_stride, out_col, H, Dv, total);
    else
        return KVB_ERR_DTYPE;
    return kvb_launch_status();
}

// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ int token_of(const int* ids, const int* src, const int* last, int r) {
    const int from = src ? src[r] : -1;
    return from >= 0 ? last[from] : ids[r];
}

// One block per row.  A token outside the vocabulary adds nothing (the embedding kernel has flagged it).
template <typename T>
__global__ void bigram_embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, const int* __restrict__ src,
                                    const int* __restrict__ last, const int* __restrict__ positions,
                                    const int* __restrict__ row_segment, const int* __restrict__ seg_q_start,
                                    const int* __restrict__ seg_slot, const int* __restrict__ previous, float* __restrict__ h,
                                    int W, int buckets, int mul_prev, int mul_cur, int V) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int tok = token_of(ids, src, last, r);
    if (tok < 0 || tok >= V) return;
    int row = buckets;
    if (positions[r] > 0) {
        const int seg = row_segment[r];
        const int before = r > seg_q_start[seg] ? token_of(ids, src, last, r - 1) : previous[seg_slot[seg]];
        row = (int)(((long long)before * mul_prev + (long long)tok * mul_cur) % buckets);
        if (row < 0) row += buckets;
    }
    const T* add = table + (size_t)row * W;
    float* dst = h + (size_t)r * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) dst[i] += to_f32<T>(add[i]);
}

__global__ void previous_token_kernel(const int* __restrict__ ids, const int* __restrict__ src, const int* __restrict__ last,
                                      const int* __restrict__ seg_q_start, const int* __restrict__ seg_q_len,
                                      const int* __restrict__ seg_slot, int* __restrict__ previous, int S) {
    pdl_wait();
    pdl_launch_dependents();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s < S && seg_q_len[s] > 0) previous[seg_slot[s]] = token_of(ids, src, last, seg_q_start[s] + seg_q_len[s] - 1);
}

KVB_API int kvb_bigram_embed(int dtype, const void* table, const int* ids, const int* src, const int* last, const int* positions,
                             const int* row_segment, const int* seg_q_start, const int* seg_q_len, const int* seg_slot,
                             int* previous, float* h, int T, int S, int W, int buckets, int mul_prev, int mul_cur, int V,
                             cudaStream_t stream) {
    if (T <= 0) return KVB_OK;
    if (buckets < 1 || W < 1) return KVB_ERR_SHAPE;
    const int threads = W >= 512 ? 256 : 128;
    if (dtype == KVB_F32)
        kvb_launch(bigram_embed_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)table, ids, src, last, positions,
                   row_segment, seg_q_start, seg_slot, previous, h, W, buckets, mul_prev, mul_cur, V);
    else if (dtype == KVB_BF16)
        kvb_launch(bigram_embed_kernel<bf16>, dim3(T), dim3(threads), 0, stream, (const bf16*)table, ids, src, last, positions,
                   row_segment, seg_q_start, seg_slot, previous, h, W, buckets, mul_prev, mul_cur, V);
    else
        return KVB_ERR_DTYPE;
    int status = kvb_launch_status();
    if (status != KVB_OK) return status;
    kvb_launch(previous_token_kernel, dim3((S + 127) / 128), dim3(128), 0, stream, ids, src, last, seg_q_start, seg_q_len, seg_slot,
               previous, S);
    return kvb_launch_status();
}
