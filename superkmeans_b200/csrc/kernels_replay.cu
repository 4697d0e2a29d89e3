// Exact replay of the pruned search for the points whose best candidate moves.
//
// The optimistic chain pass (kernels_tc_sparse.cu) leaves, for every point it flags, the short list of centroids that
// passed the first test under the starting threshold and ended below the distance to the previous centroid.  No other
// centroid can lower `best` at any time: `best` only decreases, so whatever passes a later, stricter test also passed
// the starting one, and a centroid that ends at or above the starting `best` never wins.  The search of
// BatchComputer::FindNearestNeighborWithPruning (batch_computers.h:297-409) for such a point is therefore decided by
// these candidates alone: chunk after chunk of 1024 centroids, a candidate survives when its partial distance stays
// below best * ratio[dimensions seen] at every checkpoint of PDXearch::Prune (pdxearch.h:149-216) with the `best` the
// chunk started from, and the chunk's nearest survivor replaces `best` when it is nearer.  One warp replays that for
// one point with fp32 distances from direct differences, and leaves the first-test threshold of every chunk, from
// which a counting pass over the first d' dimensions recomputes the point's not-pruned count.
#include <cfloat>
#include <cstdint>
#include <stdexcept>

#include "common.cuh"
#include "device_utils.cuh"

namespace skmb {

namespace {

__device__ __forceinline__ uint32_t warp_min_u32(uint32_t v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

}  // namespace

// meta[row]: bits 0..7 candidates recorded by the row's first thread, bits 8..15 by its second, bit 16 set when either
// found more than `cap`.  cand[(row * 2 + h) * cap + i]: global centroid index.
__global__ void __launch_bounds__(256) replay_candidates_kernel(ReplayParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t i = static_cast<size_t>(blockIdx.x) * 8 + warp;
    if (i >= p.n_listed) return;
    const size_t row = p.idx[i];
    const float best0 = p.best_in[row];
    const uint32_t prev = p.prev[row];
    const uint32_t meta = p.meta[row];
    const uint32_t c0 = meta & 0xFFu, c1 = (meta >> 8) & 0xFFu;
    const bool overflow = ((meta >> 16) & 1u) != 0 || c0 + c1 > 32u;
    const uint32_t n_chunks = static_cast<uint32_t>((p.k + kChunk - 1) / kChunk);
    const float r_first = __ldg(p.ratios + p.partial_d);
    float* thr = p.thr + i * n_chunks;
    if (overflow) {
        // too many candidates for the lists: the chain kernel redoes this point; any threshold will do meanwhile
        for (uint32_t c = lane; c < n_chunks; c += 32) thr[c] = best0 * r_first;
        if (lane == 0) p.overflow[i] = 1u;
        return;
    }
    // this lane's candidate, or none
    uint32_t mine = 0xFFFFFFFFu;
    if (static_cast<uint32_t>(lane) < c0) mine = p.cand[(row * 2 + 0) * p.cap + lane];
    else if (static_cast<uint32_t>(lane) < c0 + c1) mine = p.cand[(row * 2 + 1) * p.cap + (lane - c0)];

    const float* x = p.x + row * p.d;
    const uint32_t n_h = p.horizontal_d / 64u;
    const bool has_tail = p.partial_d < p.vertical_d;

    float best = best0;
    uint32_t best_idx = prev;
    // first-test `best` of the chunks this lane owns (lane, lane + 32)
    float bc_a = best0, bc_b = best0;
    uint32_t cur_chunk = 0xFFFFFFFFu;
    float chunk_best = FLT_MAX;
    uint32_t chunk_idx = 0;
    auto close_chunk = [&]() {
        if (cur_chunk != 0xFFFFFFFFu && chunk_best < best) {
            best = chunk_best;
            best_idx = chunk_idx;
            if (static_cast<uint32_t>(lane) > cur_chunk) bc_a = best;
            if (static_cast<uint32_t>(lane) + 32u > cur_chunk) bc_b = best;
        }
        chunk_best = FLT_MAX;
    };
    while (true) {
        const uint32_t col = warp_min_u32(mine);   // candidates in ascending order: the order of the chunks
        if (col == 0xFFFFFFFFu) break;
        if (mine == col) mine = 0xFFFFFFFFu;
        const uint32_t chunk = col / kChunk;
        if (chunk != cur_chunk) {
            close_chunk();
            cur_chunk = chunk;
        }
        const float* c = p.y + static_cast<size_t>(col) * p.d;
        // partial distances along the checkpoints, each tested against the chunk's starting `best`
        float cum = 0.f;
        bool alive = true;
        {
            float s = 0.f;
            for (uint32_t j = lane; j < p.partial_d; j += 32) {
                const float df = __ldg(x + j) - __ldg(c + j);
                s = fmaf(df, df, s);
            }
            cum = warp_sum(s);
            alive = cum < best * r_first;
        }
        uint32_t seen = p.partial_d;
        for (uint32_t h = 0; h < n_h && alive; ++h) {
            const uint32_t j0 = p.vertical_d + h * 64u;
            const float d0 = __ldg(x + j0 + lane) - __ldg(c + j0 + lane);
            const float d1 = __ldg(x + j0 + 32 + lane) - __ldg(c + j0 + 32 + lane);
            cum += warp_sum(fmaf(d0, d0, d1 * d1));
            seen += 64u;
            // the last checkpoint of all is the final distance, compared with `best` itself (ratio[d] = 1)
            if (h + 1 < n_h || has_tail) alive = cum < best * __ldg(p.ratios + seen);
        }
        if (alive && has_tail) {
            float s = 0.f;
            for (uint32_t j = p.partial_d + lane; j < p.vertical_d; j += 32) {
                const float df = __ldg(x + j) - __ldg(c + j);
                s = fmaf(df, df, s);
            }
            cum += warp_sum(s);
        }
        if (alive && cum < chunk_best) {   // strict: the first of equal distances stays, as in a scan by index
            chunk_best = cum;
            chunk_idx = col;
        }
    }
    close_chunk();
    if (static_cast<uint32_t>(lane) < n_chunks) thr[lane] = bc_a * r_first;
    if (static_cast<uint32_t>(lane) + 32u < n_chunks) thr[lane + 32] = bc_b * r_first;
    if (lane == 0) {
        p.overflow[i] = 0u;
        if (best_idx != prev) {
            p.knn[row] = best_idx;
            p.dist[row] = best;
        }
    }
}

void launch_replay_candidates(const ReplayParams& p, cudaStream_t stream) {
    if (p.n_listed == 0) return;
    if (p.k > 64 * static_cast<size_t>(kChunk)) throw std::invalid_argument("the candidate replay covers at most 64 chunks of centroids");
    if (p.cap > 16) throw std::invalid_argument("the candidate replay reads at most 16 candidates per list");
    replay_candidates_kernel<<<static_cast<unsigned>((p.n_listed + 7) / 8), 256, 0, stream>>>(p);
    SKM_LAUNCH_CHECK();
}

// out[idx[i]] = in[i]
__global__ void scatter_u32_kernel(const uint32_t* __restrict__ idx, const uint32_t* __restrict__ in, uint32_t* __restrict__ out, size_t n) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[idx[i]] = in[i];
}

void launch_scatter_u32(const uint32_t* idx, const uint32_t* in, uint32_t* out, size_t n, cudaStream_t stream) {
    if (n == 0) return;
    scatter_u32_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(idx, in, out, n);
    SKM_LAUNCH_CHECK();
}

// out[i] = outer[inner[i]]
__global__ void compose_u32_kernel(const uint32_t* __restrict__ outer, const uint32_t* __restrict__ inner, uint32_t* __restrict__ out, size_t n) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = outer[inner[i]];
}

void launch_compose_u32(const uint32_t* outer, const uint32_t* inner, uint32_t* out, size_t n, cudaStream_t stream) {
    if (n == 0) return;
    compose_u32_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(outer, inner, out, n);
    SKM_LAUNCH_CHECK();
}

}  // namespace skmb
