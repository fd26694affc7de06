// C ABI of the library (include/b200_gemm.h): validation, TMA descriptor encoding, launches,
// the host-buffer session and the seeded input generator. No CPU fallback exists: without an
// sm_100 device every compute entry point returns an error status.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>

#include "../../include/b200_gemm.h"
#include "gemm_sm100.cuh"
#include "ptx_sm100.cuh"
#include "schedule.h"
#include "synth.h"

namespace b200 {
namespace {

thread_local int t_last_cuda_error = 0;
std::atomic<uint64_t> g_wait_budget_ns{2000000000ull};
std::atomic<unsigned int> g_tail_epoch{0u};
std::atomic<long long *> g_prof_ptr{nullptr};
std::atomic<int> g_prof_blocks{0};

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct DeviceInfo {
    int ready = 0;  // 0 = not probed, 1 = usable, -1 = unusable
    int status = B200_UNSUPPORTED_DEVICE;
    int num_sms = 0;
};

constexpr int kMaxDevices = 64;
DeviceInfo g_devices[kMaxDevices];
std::mutex g_mutex;
EncodeTiledFn g_encode = nullptr;

int fail_cuda(cudaError_t e) {
    t_last_cuda_error = static_cast<int>(e);
    return B200_CUDA_ERROR;
}
}  // namespace

// For the library's other translation units: remember the CUDA error behind a B200_CUDA_ERROR
// return so that b200_last_cuda_error() reports it.
int record_cuda_error(int cuda_error) { return fail_cuda(static_cast<cudaError_t>(cuda_error)); }

namespace {

// First call on a device: check the architecture, resolve the driver's tensor-map encoder and
// opt the kernels into large dynamic shared memory.
int device_info(const DeviceInfo **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail_cuda(e);
    if (dev < 0 || dev >= kMaxDevices) return B200_UNSUPPORTED_DEVICE;
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceInfo &d = g_devices[dev];
    if (d.ready == 0) {
        d.ready = -1;
        cudaDeviceProp prop;
        e = cudaGetDeviceProperties(&prop, dev);
        if (e != cudaSuccess) {
            d.status = fail_cuda(e);
            return d.status;
        }
        if (prop.major != 10) {
            d.status = B200_UNSUPPORTED_DEVICE;
            return d.status;
        }
        d.num_sms = prop.multiProcessorCount;
        if (!g_encode) {
            void *fn = nullptr;
            cudaDriverEntryPointQueryResult qres;
            e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
            if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
                d.status = fail_cuda(e != cudaSuccess ? e : cudaErrorUnknown);
                return d.status;
            }
            g_encode = reinterpret_cast<EncodeTiledFn>(fn);
        }
        const int pe = prepare_kernels();
        if (pe != 0) {
            d.status = fail_cuda(static_cast<cudaError_t>(pe));
            return d.status;
        }
        d.status = B200_OK;
        d.ready = 1;
    }
    *out = &d;
    return d.status;
}

int encode_2d(CUtensorMap *map, CUtensorMapDataType type, int elem_bytes, const void *ptr, uint64_t inner,
              uint64_t outer, uint32_t box_inner, uint32_t box_outer, uint64_t pitch_elems = 0) {
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {(pitch_elems ? pitch_elems : inner) * static_cast<uint64_t>(elem_bytes)};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = g_encode(map, type, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        t_last_cuda_error = static_cast<int>(cudaErrorInvalidValue);
        return B200_CUDA_ERROR;
    }
    return B200_OK;
}

// Tuned defaults. Large problems use the two-CTA pair (256 x 256 tile, each CTA stages 128 rows of
// A and 128 rows of B^T per K block: half the L2-to-shared traffic per flop of a one-CTA
// 128 x 256 tile); small or skinny ones a one-CTA tile with the widest N that divides.
void default_params(int64_t M, int64_t N, int64_t K, b200_gemm_params *p, bool allow_swap = true, bool allow_tall = true) {
    std::memset(p, 0, sizeof(*p));
    // The two-CTA 256 x 256 tile needs enough tiles to occupy the GPU: below half of the 74 pairs
    // (1024^2 has 16) narrower one-CTA tiles finish sooner (1024^3: 7.3 against 11.3 us).
    const bool pair = (M > 128) && (N % 256 == 0) && ((M + 255) / 256) * (N / 256) >= 37;
    const int64_t n_tiles128 = (N + 127) / 128;
    const bool few_tiles = K >= 4096 && n_tiles128 <= 74;
    if (allow_swap && (M <= 64 || (M <= 128 && few_tiles))) {
        // Decode shapes: the weights are the whole traffic. Swapped roles stage 128 weight rows and
        // only the activation rows there are per K block; 128-deep K segments halve the barrier
        // round trips per byte. One SM sustains a few tens of GB/s of TMA loads at DRAM latency, so
        // when there are few tiles their K range is split over a cluster to put more SMs to work
        // (measured: 4 slices beat 2 even at 56 tiles; beyond 64 rows the swapped form is used only with the cluster split).
        p->swap_ab = 1;
        p->tile_m = static_cast<int>((M + 15) / 16 * 16);
        p->tile_n = 128;
        p->cta_group = 1;
        p->segment_dim_k = M <= 64 ? 128 : 64;
        p->num_stages = M <= 32 ? 5 : (M <= 64 ? 4 : 5);
        p->num_producer_warps = 1;
        p->l2_hint = 1;
        p->bar_step_rows_a = p->tile_m;
        p->bar_step_rows_b = p->tile_n;
        p->tile_group_m = 8;
        p->num_consumer_warps = 4;
        p->split_k = 1;
        if (few_tiles) {
            p->split_k = 4;
            p->cluster_reduce = 1;
        } else if (n_tiles128 > 148) {
            // an even share of tiles per CTA (224 tiles: 112 CTAs x 2 rather than 76 x 2 + 72 x 1; +1.5 %)
            const int64_t waves = (n_tiles128 + 147) / 148;
            p->num_sms = static_cast<int>((n_tiles128 + waves - 1) / waves);
        }
        // A short kernel: let set-up overlap the previous kernel of the stream (measured -4 % on the
        // 4- and 8-GPU shards of the decode shape, 117 and 59 MB of weights; +6 % on the whole one,
        // 470 MB, where all SMs are busy for 70 us).
        p->overlap_launch = (N * K * 2 <= 160000000) ? 1 : 0;
        if (M > 64 && few_tiles && N >= 256) {
            // 65 - 128 activation rows and few tiles: the swapped pair (256 weight rows per tile, each CTA stages 128 of
            // them and half of the activation rows) over a cluster of four pairs, and eight draining warps, which
            // halve the staging and the reduce of the 128-column accumulator (tuner, interleaved: 128 x 7168: 27.1
            // against 28.4 us for the 4-CTA form with four warps; 128 x 3584: 18.2 against 18.9 us)
            p->tile_m = static_cast<int>((M + 31) / 32 * 32);
            p->tile_n = 256;
            p->cta_group = 2;
            p->segment_dim_k = 64;
            p->num_stages = 6;
            p->num_consumer_warps = 8;
            p->bar_step_rows_a = p->tile_m;
            p->bar_step_rows_b = p->tile_n;
        }
        return;
    }
    if (allow_swap && M > 64 && M <= 128 && n_tiles128 >= 112) {
        // 65 - 128 activation rows against many weight rows: the swapped two-CTA pair. Each CTA stages
        // 128 weight rows and half of the activation rows per K block (measured 2 - 3 % over the plain
        // 128 x 224 tile at N = 14336 and 28672; below that the plain narrow tiles fill more SMs).
        p->swap_ab = 1;
        p->tile_m = static_cast<int>((M + 31) / 32 * 32);
        p->tile_n = 256;
        p->cta_group = 2;
        p->segment_dim_k = 64;
        p->num_stages = 8;
        p->num_producer_warps = 1;
        p->l2_hint = 1;
        p->bar_step_rows_a = p->tile_m;
        p->bar_step_rows_b = p->tile_n;
        p->tile_group_m = 8;
        p->num_consumer_warps = 4;
        p->split_k = 1;
        // an even share of pair tiles per CTA pair (112 tiles: 56 pairs x 2 rather than 38 x 2 + 36 x 1; +0.8 %)
        const int64_t pair_tiles = (N + 255) / 256;
        if (pair_tiles > 74) {
            const int64_t waves = (pair_tiles + 73) / 74;
            p->num_sms = static_cast<int>(2 * ((pair_tiles + waves - 1) / waves));
        }
        return;
    }
    bool tall = false;
    if (pair) {
        p->tile_m = 256;
        p->cta_group = 2;
        // Tile width against wave quantisation: 74 CTA pairs run a wave of tiles, and a last wave that is partly
        // empty still costs a whole tile time. Narrower tiles (224 or 192 columns, the last tile column ragged
        // where they do not divide N) can make the waves come out even - 1024 x 8192: 4 x 37 tiles of 224 columns
        // are exactly two waves, where 4 x 32 tiles of 256 take two waves of which the second is 73 % full -
        // at the price of more operand traffic per flop. Cost = waves x (columns + a per-tile charge). The 256-column
        // tile is credited with the tail split's saving where that applies (measured: 4096^3 and 2048 x 8192 x 8192
        // run faster with 256 columns and the tail cut in two than with 224 or 192 columns); a narrower tile has to
        // win by 3 % without it, since the tail split only engages when the caller passes a workspace.
        const int64_t rows = (M + 255) / 256;
        int best_n = 256;
        double best_cost = 0.0;
        for (int tn = 256; tn >= 192; tn -= 32) {
            const int64_t tiles = rows * ((N + tn - 1) / tn);
            const int64_t full = tiles / 74, r = tiles % 74;
            double waves = double(full);
            if (r > 0) {
                const int64_t s = 74 / r > 8 ? 8 : 74 / r;
                waves += (tn == 256 && s >= 2 && K / 64 / s >= 4) ? 1.0 / double(s) + 0.04 : 1.0;
            }
            const double cost = waves * double(tn + 12) * (tn == 256 ? 1.0 : 1.02);
            if (tn == 256 || cost < best_cost * 0.97) {
                best_cost = cost;
                best_n = tn;
            }
        }
        p->tile_n = best_n;
        p->num_stages = 6;   // 6 x (128 + tile_n / 2) rows x 128 B, and 32 KB of TMA-store staging: 224 KB with 256 columns
        p->num_producer_warps = 2;
        p->l2_hint = 3;  // keep operand panels in L2: fewer DRAM re-reads, measured +2.5 % under the power limit
        // The tall pair (512 x 256 per pair, 256 rows of A per CTA as two MMA atoms against one B^T stage) moves a
        // quarter fewer operand bytes per flop from L2 to the SMs: the K loop stops waiting for data (1049 against
        // 1106 cycles per 512 x 256 x 64 block) and a launch costs less energy, which under the power limit is clock.
        // Its accumulators fill the tensor memory, so the drain of a tile (9.5 k cycles with eight warps) is not
        // hidden behind the next tile's MMAs: 7 % of a tile at K = 8192, more at smaller K. Measured at 8192^3:
        // 1491 against 1443 TFLOP/s (0.968 of the time). Taken when its rounds cost less by that model, in the width
        // that makes its rounds come out even: 224 columns for the row shards of 8192^3 (1024 x 8192: 2 x 37 tiles are
        // exactly one round, +4.4 % over two waves of 256 x 224 pairs; 2048 and 4096 rows: two and four rounds, +3.8 %
        // and +1.4 %), 256 for the whole of it (7 rounds of 74).
        if (K >= 4096 && allow_tall) {
            const double tall_factor = 0.968 + 0.071 * (8192.0 / double(K) - 1.0);
            for (int tn = 256; tn >= 192; tn -= 32) {
                const int64_t tall_tiles = ((M + 511) / 512) * ((N + tn - 1) / tn);
                const int64_t tall_rounds = (tall_tiles + 73) / 74;
                const double tall_cost = double(tall_rounds) * 2.0 * double(tn + 12) * tall_factor * (tn == 256 ? 1.0 : 1.01);
                if (tall_cost < best_cost * 0.995) {
                    best_cost = tall_cost / 0.995;   // a narrower tall tile has to beat this one in turn
                    best_n = tn;
                    tall = true;
                }
            }
            if (tall) p->tile_n = best_n;
        }
    } else {
        // One row of tiles (skinny, HBM-bound: decode shapes) or N not a multiple of 256: a one-CTA
        // tile whose width divides N and fills the last wave of the persistent grid best.
        p->tile_m = 128;
        p->cta_group = 1;
        int best_n = 16;
        double best_eff = -1.0;
        const int64_t rows = (M + 127) / 128;
        for (int tn = 256; tn >= 16; tn -= 16) {
            if (N % tn) continue;
            const int64_t tiles = rows * (N / tn);
            const int64_t waves = (tiles + 147) / 148;
            // narrow tiles cost tensor-core efficiency, which only matters when the shape is not HBM-bound
            // (nor when the whole problem is less than one wave of 128 x 128 tiles: then it is latency-bound)
            const bool small = rows * ((N + 127) / 128) < 148;
            const double eff = double(tiles) / double(waves * 148) *
                               ((tn >= 128 || (M <= 128 && tn >= 32) || (small && tn >= 64)) ? 1.0 : tn / 128.0);
            if (eff > best_eff + 1e-9) {
                best_eff = eff;
                best_n = tn;
            }
        }
        if (best_eff < 0.0) best_n = 128;  // no width divides N: ragged last tile column
        p->tile_n = best_n;
        const int stage_bytes = (128 + best_n) * 128;
        p->num_stages = 198000 / stage_bytes > 8 ? 8 : 198000 / stage_bytes;  // leaves room for the TMA-store staging
        p->num_producer_warps = 1;
        // weights stream through once (evict_first), the few activation rows are re-read by every CTA
        p->l2_hint = (M <= 128) ? 1 : 3;
    }
    p->segment_dim_k = 64;
    p->bar_steps_a = 0;
    p->bar_steps_b = 0;
    p->bar_step_rows_a = p->tile_m;  // shift synchronisation off
    p->bar_step_rows_b = p->tile_n;
    p->tile_group_m = 8;
    if (pair) {
        // Operand panels are re-read from DRAM by every wave of 74 tile pairs (a wave's panels, 69 MB at K = 8192,
        // are more than the L2 keeps from one wave to the next). Walking K downwards in every other tile of a CTA
        // hands the next wave the panel ends touched last while they are still in L2, and groups of 16 tile rows
        // halve the number of times a B^T panel is fetched: DRAM reads 1.15 -> 0.95 GB per 8192^3 launch, which
        // under the power limit is +2.7 % (1486 against 1447 TFLOP/s, interleaved on one GPU; groups of 8 / 12 / 20 /
        // 24 / 32 rows with the same K order: 1464 / 1473 / 1466 / 1451 / 1420).
        p->k_order = 1;
        p->tile_group_m = 16;
    }
    p->num_consumer_warps = 4;
    if (tall) {
        p->tile_m = 512;
        p->bar_step_rows_a = 512;
        p->bar_step_rows_b = p->tile_n;
        // 256 columns: 3 x 48 KB of stages + 64 KB of drain buffers (two boxes for each of eight warps); narrower: a
        // fourth stage pays (919 against 1009 cycles per K block at 224 columns) and the warps stage through one box each
        p->num_stages = p->tile_n == 256 ? 3 : 4;
        p->num_consumer_warps = 8;  // the drain is exposed: two warps per tensor-memory lane quarter halve it
        p->tile_group_m = 8;        // 8 x 512 rows: the same 4096-row groups as 16 x 256
    }
    p->num_sms = 0;
    p->split_k = 1;
    // drain through swizzled shared memory and TMA stores: 3x shorter per tile than scattered 128-bit
    // stores (6.2 k vs 19 k cycles for 128 x 256 fp32), +2 % on 8192^3
    p->epilogue = 1;
    // tiles that do not fill a wave are scheduled by K iterations (takes effect when the call gets a workspace)
    p->tail_split = 1;
    // a grid that leaves SMs idle is a short kernel: overlap its set-up with the previous kernel's tail
    const int64_t ctas = ((M + p->tile_m - 1) / p->tile_m) * ((N + p->tile_n - 1) / p->tile_n) * p->cta_group;
    p->overlap_launch = ctas < 148 ? 1 : 0;
}

struct PushTarget {  // split-K over GPUs with the exchange fused into the epilogue; world == 0: off
    int world = 0, rank = 0, epoch = 0;
    void *const *slots = nullptr;
    void *const *flags = nullptr;
    void *done = nullptr;
};

int gemm_impl(int dtype, const void *A, const void *Bt, const float *C, float *D, float alpha, float beta, int64_t M,
              int64_t N, int64_t K, const b200_gemm_params *user, void *workspace, size_t workspace_bytes,
              cudaStream_t stream, const PushTarget *push = nullptr, int64_t ld_cd = 0, bool out_half = false) {
    // out_half: C and D point to fp16 matrices (passed through the float pointers unread on the host)
    if (dtype != B200_F16 && dtype != B200_BF16) return B200_INVALID_CONFIG;
    b200_gemm_params local;
    if (!user) {
        // The tall pair's drain is exposed; it pays only through the lean TMA-store drain of beta = 0 (with C to read the
        // drain takes half as long again: 8192^3 at beta = 1 1.0 - 1.26 against 1.23 - 1.41 PFLOP/s for the 256-row pair,
        // whose drain hides behind the next tile), which fp16 output and a push target do not have either: those keep
        // the 256-row pair.
        default_params(M, N, K, &local, true, !(out_half || beta != 0.0f || (push && push->world > 0)));
        user = &local;
    }
    const DeviceInfo *dev = nullptr;
    int st = device_info(&dev);
    if (st != B200_OK) return st;
    const Plan p = make_plan(*user, dev->num_sms);
    if (p.status != B200_OK) return p.status;
    st = check_shape(p, M, N, K);
    if (st != B200_OK) return st;
    const bool pushing = push && push->world > 0;
    if ((p.swap || p.atoms > 1) && pushing) return B200_INVALID_CONFIG;
    // Swapped roles: the kernel sees the transposed problem (its M operand is B^T, its N operand A)
    // and writes its accumulator transposed, so C and D keep their row-major m x n layout.
    const int64_t kM = p.swap ? N : M, kN = p.swap ? M : N;
    const void *const opA = p.swap ? Bt : A;
    const void *const opB = p.swap ? A : Bt;
    if (pushing) {
        if (push->world > 8 || push->rank < 0 || push->rank >= push->world || !push->slots || !push->flags || !push->done)
            return B200_INVALID_CONFIG;
        if (M % push->world || (M / push->world) % 128 || (M / push->world) % p.cta_rows_a || N % 4)
            return B200_INVALID_SHAPE;  // every CTA's rows must belong to one owner
        for (int o = 0; o < push->world; ++o)
            if (!push->slots[o] || !push->flags[o]) return B200_INVALID_POINTER;
    }
    if (!A || !Bt || (!D && !pushing)) return B200_INVALID_POINTER;
    if (beta != 0.0f && !C) return B200_INVALID_POINTER;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(Bt) | reinterpret_cast<uintptr_t>(D) |
         reinterpret_cast<uintptr_t>(C)) & 15u)
        return B200_INVALID_POINTER;
    const int64_t n_tiles = ((kM + p.tile_m - 1) / p.tile_m) * ((kN + p.tile_n - 1) / p.tile_n);
    // The tail split is an optimisation of the schedule, taken when the caller's workspace can hold the partials;
    // without it the plain schedule runs and the result is the same to rounding. Its CTAs wait for one another,
    // so all of them must be resident at once: one per SM.
    TailPlan tail = make_tail_plan(user->tail_split && !p.swap && p.atoms == 1 && p.grid <= dev->num_sms, n_tiles, p.grid / p.cta_group,
                                   (K + p.seg_k - 1) / p.seg_k, p.split_k, p.tile_n, p.cta_group);
    if (tail.tiles > 0 && (!workspace || workspace_bytes < static_cast<size_t>(tail.slot_bytes * tail.slots) ||
                           (reinterpret_cast<uintptr_t>(workspace) & 15u)))
        tail = TailPlan();
    const int ws_split = p.cluster_reduce ? 1 : p.split_k;  // K slices that meet in the workspace
    // fp16 output leaves through the plain, transposed and cluster drains only: the split-K workspace and
    // push forms keep fp32 partials and their second kernels write fp32
    if (out_half && (ws_split > 1 || pushing)) return B200_INVALID_CONFIG;
    if (ld_cd && ld_cd != N && (ws_split > 1 || (push && push->world > 0) || ld_cd < N || ld_cd % 4))
        return B200_INVALID_CONFIG;  // the second-step kernels assume a dense D
    if (ws_split > 1) {
        const size_t need = static_cast<size_t>(p.split_k) * static_cast<size_t>(M) * static_cast<size_t>(N) * sizeof(float);
        if (!workspace || workspace_bytes < need) return B200_WORKSPACE_TOO_SMALL;
        if (reinterpret_cast<uintptr_t>(workspace) & 15u) return B200_INVALID_POINTER;
    }

    GemmArgs a;
    std::memset(&a, 0, sizeof(a));
    const CUtensorMapDataType in_type = dtype == B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    st = encode_2d(&a.map_a, in_type, 2, opA, static_cast<uint64_t>(K), static_cast<uint64_t>(kM), kBoxK,
                   static_cast<uint32_t>(p.a_box_rows));
    if (st != B200_OK) return st;
    st = encode_2d(&a.map_b, in_type, 2, opB, static_cast<uint64_t>(K), static_cast<uint64_t>(kN), kBoxK,
                   static_cast<uint32_t>(p.chunk_n / p.cta_group));
    if (st != B200_OK) return st;
    int epi_mode = p.epi_mode;
    if (p.mma_m != 128 || ws_split > 1 || pushing || out_half) epi_mode = 0;  // the TMA-store drain needs 32 consecutive rows per warp
    if (epi_mode) {
        st = encode_2d(&a.map_d, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, D, static_cast<uint64_t>(N), static_cast<uint64_t>(M),
                       kEpiBoxCols, 32, static_cast<uint64_t>(ld_cd));
        if (st != B200_OK) return st;
    }
    a.C = C;
    a.D = D;
    a.partial = static_cast<float *>(workspace);
    a.alpha = alpha;
    a.beta = beta;
    a.M = static_cast<int>(kM);
    a.N = static_cast<int>(kN);
    a.K = static_cast<int>(K);
    a.swap_ab = p.swap;
    a.out_half = out_half ? 1 : 0;
    a.ld_cd = static_cast<int>(ld_cd ? ld_cd : N);
    a.tiles_m = static_cast<int>((kM + p.tile_m - 1) / p.tile_m);
    a.tiles_n = static_cast<int>((kN + p.tile_n - 1) / p.tile_n);
    a.num_tiles = a.tiles_m * a.tiles_n;
    a.split_k = ws_split;
    a.cl_split = p.cluster_reduce ? p.split_k : 0;
    a.num_units = a.num_tiles * ws_split;
    a.tail_tiles = tail.tiles;
    a.tail_slices = tail.slices;
    if (tail.tiles > 0) {
        // every launch that uses the fix-up flags gets its own epoch (never 0) and the next flag set in turn
        unsigned int epoch = g_tail_epoch.fetch_add(1u) + 1u;
        if (epoch == 0u) epoch = g_tail_epoch.fetch_add(1u) + 1u;
        a.tail_epoch = epoch;
        a.tail_set = static_cast<int>(epoch & 0x7fffffffu);
    }
    a.num_segs = static_cast<int>((K + p.seg_k - 1) / p.seg_k);
    a.tile_m = p.tile_m;
    a.tile_n = p.tile_n;
    a.cta_rows_a = p.cta_rows_a;
    a.mma_m = p.mma_m;
    a.kblocks = p.kblocks;
    a.stages = p.stages;
    a.tile_group_m = p.tile_group_m;
    a.a_box_rows = p.a_box_rows;
    a.a_boxes = p.a_boxes;
    a.a_priv = p.a_priv;
    a.a_bars = p.a_bars;
    a.chunk_n = p.chunk_n;
    a.b_priv = p.b_priv;
    a.b_res_chunks = p.b_res_chunks;
    a.b_bars = p.b_bars;
    a.producer_warps = p.producer_warps;
    a.epi_warps = p.epi_warps;
    a.acc_cols = p.acc_cols;
    a.tmem_cols = p.tmem_cols;
    a.a_stage_bytes = p.a_stage_bytes;
    a.stage_bytes = p.stage_bytes;
    a.off_epi = p.off_epi;
    a.off_bars = p.off_bars;
    a.off_tmem_ptr = p.off_tmem_ptr;
    a.epi_mode = epi_mode;
    const int atom_m = p.cta_group * p.mma_m;   // M of one MMA (the pair's 256 spans both CTAs)
    a.idesc_chunk = umma_idesc(atom_m, p.chunk_n, dtype == B200_BF16);
    a.idesc_res = umma_idesc(atom_m, p.b_res_chunks * p.chunk_n, dtype == B200_BF16);
    a.a_split = p.a_split;
    a.atoms = p.atoms;
    a.epi_bufs = p.epi_bufs;
    a.wait_budget_cycles = static_cast<long long>(g_wait_budget_ns.load() * 2ull);  // SM clock is below 2 GHz

    if (pushing && ws_split == 1) {
        for (int o = 0; o < push->world; ++o) {
            a.push_slot[o] = static_cast<float *>(push->slots[o]);
            a.push_flag[o] = static_cast<int *>(push->flags[o]);
        }
        a.push_done = static_cast<unsigned int *>(push->done);
        a.push_world = push->world;
        a.push_rank = push->rank;
        a.push_rows = static_cast<int>(M / push->world);
        a.push_epoch = push->epoch;
    }
    a.prof = g_prof_ptr.load();
    a.prof_blocks = g_prof_blocks.load();
    a.debug_flags = user->diagnostic;
    a.l2_hint = user->l2_hint;
    // D larger than half the L2 (126 MB) streams out with evict_first lines; bit 5 of the diagnostic word keeps them normal
    a.d_stream = (static_cast<int64_t>(M) * N * (out_half ? 2 : 4) >= (int64_t(64) << 20)) && !(user->diagnostic & 32);
    a.k_order = user->k_order;
    a.overlap_launch = user->overlap_launch ? 1 : 0;

    const int le = launch_gemm(p, a, stream);
    if (le != 0) return fail_cuda(static_cast<cudaError_t>(le));
    if (ws_split > 1 && pushing) {
        float *slots[8];
        int *flags[8];
        for (int o = 0; o < push->world; ++o) {
            slots[o] = static_cast<float *>(push->slots[o]);
            flags[o] = static_cast<int *>(push->flags[o]);
        }
        const int re = launch_splitk_reduce_push(a.partial, M, N, p.split_k, slots, flags, static_cast<unsigned int *>(push->done),
                                                 push->world, push->rank, push->epoch, stream);
        if (re != 0) return fail_cuda(static_cast<cudaError_t>(re));
    } else if (ws_split > 1) {
        const int re = launch_splitk_reduce(a.partial, C, D, alpha, beta, M * N, p.split_k, stream);
        if (re != 0) return fail_cuda(static_cast<cudaError_t>(re));
    }
    return B200_OK;
}

__global__ void fill_u16_kernel(uint16_t *dst, long long begin, long long count, uint64_t key, int dist, float sigma,
                                int dtype) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
        dst[i] = synth::value_u16(key, static_cast<uint64_t>(begin + i), dist, sigma, dtype);
}

__global__ void fill_f32_kernel(float *dst, long long begin, long long count, uint64_t key, int dist, float sigma) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
        dst[i] = synth::value(key, static_cast<uint64_t>(begin + i), dist, sigma);
}

}  // namespace
}  // namespace b200

using namespace b200;

constexpr int kSessionEvents = 16;   // two per upload step of the host-buffer call (up to eight steps)

struct b200_session {
    int64_t max_m, max_n, max_k;
    void *dA, *dB;
    float *dC, *dD;
    cudaStream_t stream;      // uploads
    cudaStream_t compute;     // launches
    cudaStream_t download;    // results
    cudaStream_t push;        // copies of this GPU's B^T rows into the other GPUs (sharded call)
    cudaEvent_t up[kSessionEvents], done[kSessionEvents], b_ready;
    void *dW;                 // workspace for the tail split of the block products
    size_t w_bytes;
};

extern "C" {

int b200_gemm_default_params(int64_t M, int64_t N, int64_t K, int dtype, b200_gemm_params *p) {
    if (!p) return B200_INVALID_POINTER;
    (void)dtype;
    default_params(M, N, K, p);
    return B200_OK;
}

int b200_gemm_default_params_for_call(int64_t M, int64_t N, int64_t K, int dtype, float beta, int fp16_out, b200_gemm_params *p) {
    if (!p) return B200_INVALID_POINTER;
    (void)dtype;
    default_params(M, N, K, p, true, !(fp16_out || beta != 0.0f));
    return B200_OK;
}

int b200_gemm_default_params_plain(int64_t M, int64_t N, int64_t K, int dtype, b200_gemm_params *p) {
    if (!p) return B200_INVALID_POINTER;
    (void)dtype;
    default_params(M, N, K, p, false);
    return B200_OK;
}

int b200_gemm_validate(int64_t M, int64_t N, int64_t K, int dtype, const b200_gemm_params *p) {
    if (!p) return B200_INVALID_POINTER;
    if (dtype != B200_F16 && dtype != B200_BF16) return B200_INVALID_CONFIG;
    const Plan plan = make_plan(*p, p->num_sms > 0 ? p->num_sms : 148);
    if (plan.status != B200_OK) return plan.status;
    return check_shape(plan, M, N, K);
}

int64_t b200_gemm_smem_bytes(int dtype, const b200_gemm_params *p) {
    (void)dtype;
    if (!p) return -1;
    const Plan plan = make_plan(*p, p->num_sms > 0 ? p->num_sms : 148);
    return plan.status == B200_OK ? plan.smem_bytes : -1;
}

int b200_gemm_schedule(int64_t M, int64_t N, int64_t K, const b200_gemm_params *p, int num_sms, int group, int *units,
                       int max_units, int *num_groups_out) {
    if (!p || num_sms <= 0) return -1;
    b200_gemm_params q = *p;
    q.num_sms = num_sms;
    const Plan plan = make_plan(q, num_sms);
    if (plan.status != B200_OK || check_shape(plan, M, N, K) != B200_OK) return -1;
    const int64_t kM = plan.swap ? N : M, kN = plan.swap ? M : N;
    Cfg c;
    std::memset(&c, 0, sizeof(c));
    c.tile_m = plan.tile_m;
    c.tile_n = plan.tile_n;
    c.tiles_m = static_cast<int>((kM + plan.tile_m - 1) / plan.tile_m);
    c.tiles_n = static_cast<int>((kN + plan.tile_n - 1) / plan.tile_n);
    c.num_tiles = c.tiles_m * c.tiles_n;
    c.tile_group_m = plan.tile_group_m;
    c.num_segs = static_cast<int>((K + plan.seg_k - 1) / plan.seg_k);
    c.split_k = plan.cluster_reduce ? 1 : plan.split_k;
    c.cl_split = plan.cluster_reduce ? plan.split_k : 1;
    c.num_units = c.num_tiles * c.split_k;
    int grid = plan.grid;
    if (plan.cluster_reduce) {                      // as launch_gemm: whole clusters, no more than there are tiles
        const int per_tile = plan.split_k * plan.cta_group;
        grid -= grid % per_tile;
        if (grid > c.num_tiles * per_tile) grid = c.num_tiles * per_tile;
        if (grid < per_tile) grid = per_tile;
    }
    const int num_groups = grid / (plan.cta_group * c.cl_split);
    if (num_groups_out) *num_groups_out = num_groups;
    if (group < 0 || group >= num_groups) return -1;
    const TailPlan tail = make_tail_plan(q.tail_split && !plan.swap && plan.atoms == 1, c.num_tiles, num_groups, c.num_segs, plan.split_k, plan.tile_n,
                                         plan.cta_group);
    c.tail_tiles = tail.tiles;
    c.tail_slices = tail.slices;
    c.cl_seg_end = c.num_segs;   // a cluster's slices: listed for slice 0 .. as the whole K range of the tile
    Walk walk;
    walk_init(c, walk, group);
    Unit w;
    int n = 0;
    while (walk_next(c, walk, num_groups, w)) {
        if (units && n < max_units) {
            int *u = units + 6 * n;
            u[0] = w.m0; u[1] = w.n0; u[2] = w.seg_begin; u[3] = w.seg_end; u[4] = w.kind; u[5] = w.slice;
        }
        ++n;
    }
    return n;
}

int64_t b200_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, const b200_gemm_params *p) {
    if (!p) return 0;
    if (p->split_k > 1 && !p->cluster_reduce) return static_cast<int64_t>(p->split_k) * M * N * static_cast<int64_t>(sizeof(float));
    if (p->tail_split) {
        int sms = p->num_sms;
        if (sms <= 0) {                        // the grid follows the device: ask it; 148 (a B200) without one
            int dev = 0, n = 0;
            sms = (cudaGetDevice(&dev) == cudaSuccess &&
                   cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 148;
            cudaGetLastError();
        }
        const Plan plan = make_plan(*p, sms);
        if (plan.status != B200_OK || plan.swap || plan.atoms > 1) return 0;
        const int64_t n_tiles = ((M + plan.tile_m - 1) / plan.tile_m) * ((N + plan.tile_n - 1) / plan.tile_n);
        const TailPlan t = make_tail_plan(1, n_tiles, plan.grid / plan.cta_group, (K + plan.seg_k - 1) / plan.seg_k, plan.split_k,
                                          plan.tile_n, plan.cta_group);
        if (t.tiles > 0) return t.slot_bytes * t.slots;
    }
    return 0;
}

int b200_gemm_f16(const void *A, const void *Bt, const float *C, float *D, float alpha, float beta, int64_t M, int64_t N,
                  int64_t K, const b200_gemm_params *p, void *workspace, size_t workspace_bytes, void *stream) {
    return gemm_impl(B200_F16, A, Bt, C, D, alpha, beta, M, N, K, p, workspace, workspace_bytes,
                     static_cast<cudaStream_t>(stream));
}

int b200_gemm_bf16(const void *A, const void *Bt, const float *C, float *D, float alpha, float beta, int64_t M, int64_t N,
                   int64_t K, const b200_gemm_params *p, void *workspace, size_t workspace_bytes, void *stream) {
    return gemm_impl(B200_BF16, A, Bt, C, D, alpha, beta, M, N, K, p, workspace, workspace_bytes,
                     static_cast<cudaStream_t>(stream));
}

int b200_gemm_f16_out_f16(const void *A, const void *Bt, const void *C, void *D, float alpha, float beta, int64_t M,
                          int64_t N, int64_t K, const b200_gemm_params *p, void *stream) {
    return gemm_impl(B200_F16, A, Bt, static_cast<const float *>(C), static_cast<float *>(D), alpha, beta, M, N, K, p, nullptr, 0,
                     static_cast<cudaStream_t>(stream), nullptr, 0, true);
}

int b200_gemm_push(int dtype, const void *A, const void *Bt, int64_t M, int64_t N, int64_t K, const b200_gemm_params *p,
                   int world, int rank, void *const *slot_ptrs, void *const *flag_ptrs, void *done_counter, int epoch,
                   void *workspace, size_t workspace_bytes, void *stream) {
    PushTarget t;
    t.world = world;
    t.rank = rank;
    t.epoch = epoch;
    t.slots = slot_ptrs;
    t.flags = flag_ptrs;
    t.done = done_counter;
    if (world < 1) return B200_INVALID_CONFIG;
    return gemm_impl(dtype, A, Bt, nullptr, nullptr, 1.0f, 0.0f, M, N, K, p, workspace, workspace_bytes,
                     static_cast<cudaStream_t>(stream), &t);
}

int b200_push_reduce(const float *my_slots, const int *my_flags, int world, int epoch, const float *C, float *D, float alpha,
                     float beta, int64_t rows, int64_t N, void *stream) {
    if (!my_slots || !my_flags || !D || world < 1 || world > 8 || rows <= 0 || N <= 0 || (rows * N) % 4) return B200_INVALID_SHAPE;
    if (beta != 0.0f && !C) return B200_INVALID_POINTER;
    const int e = launch_push_reduce(my_slots, my_flags, world, epoch, C, D, alpha, beta, rows, N,
                                     static_cast<long long>(g_wait_budget_ns.load() * 2ull), static_cast<cudaStream_t>(stream));
    return e == 0 ? B200_OK : fail_cuda(static_cast<cudaError_t>(e));
}

int b200_peer_alloc(size_t bytes, void **out) {
    if (!out || bytes == 0) return B200_INVALID_POINTER;
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
    if (e != cudaSuccess) return fail_cuda(e);
    *out = p;
    return B200_OK;
}

int b200_peer_free(void *ptr) {
    const cudaError_t e = cudaFree(ptr);
    return e == cudaSuccess ? B200_OK : fail_cuda(e);
}

int b200_peer_export(void *ptr, unsigned char handle[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    if (!ptr || !handle) return B200_INVALID_POINTER;
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
    if (e != cudaSuccess) return fail_cuda(e);
    std::memcpy(handle, &h, 64);
    return B200_OK;
}

int b200_peer_import(const unsigned char handle[64], void **out) {
    if (!handle || !out) return B200_INVALID_POINTER;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    void *p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail_cuda(e);
    *out = p;
    return B200_OK;
}

int b200_peer_release(void *imported) {
    const cudaError_t e = cudaIpcCloseMemHandle(imported);
    return e == cudaSuccess ? B200_OK : fail_cuda(e);
}

int b200_session_create(int64_t max_m, int64_t max_n, int64_t max_k, b200_session **out) {
    if (!out || max_m <= 0 || max_n <= 0 || max_k <= 0) return B200_INVALID_SHAPE;
    const DeviceInfo *dev = nullptr;
    const int st = device_info(&dev);
    if (st != B200_OK) return st;
    b200_session *s = new (std::nothrow) b200_session();
    if (!s) return B200_CUDA_ERROR;
    std::memset(s, 0, sizeof(*s));
    s->max_m = max_m;
    s->max_n = max_n;
    s->max_k = max_k;
    cudaError_t e = cudaMalloc(&s->dA, static_cast<size_t>(max_m) * max_k * 2);
    if (e == cudaSuccess) e = cudaMalloc(&s->dB, static_cast<size_t>(max_n) * max_k * 2);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&s->dC), static_cast<size_t>(max_m) * max_n * 4);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&s->dD), static_cast<size_t>(max_m) * max_n * 4);
    s->w_bytes = static_cast<size_t>(192) * 128 * 256 * sizeof(float);   // tail-split partials of the block products (a smaller need is the common case; a larger one falls back to the plain schedule)
    if (e == cudaSuccess) e = cudaMalloc(&s->dW, s->w_bytes);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&s->compute, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&s->download, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&s->push, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&s->b_ready, cudaEventDisableTiming);
    for (int i = 0; i < kSessionEvents && e == cudaSuccess; ++i) {
        e = cudaEventCreateWithFlags(&s->up[i], cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&s->done[i], cudaEventDisableTiming);
    }
    if (e != cudaSuccess) {
        b200_session_destroy(s);
        return fail_cuda(e);
    }
    *out = s;
    return B200_OK;
}

void b200_session_destroy(b200_session *s) {
    if (!s) return;
    if (s->stream) cudaStreamDestroy(s->stream);
    if (s->compute) cudaStreamDestroy(s->compute);
    if (s->download) cudaStreamDestroy(s->download);
    if (s->push) cudaStreamDestroy(s->push);
    if (s->b_ready) cudaEventDestroy(s->b_ready);
    for (int i = 0; i < kSessionEvents; ++i) {
        if (s->up[i]) cudaEventDestroy(s->up[i]);
        if (s->done[i]) cudaEventDestroy(s->done[i]);
    }
    cudaFree(s->dA);
    cudaFree(s->dB);
    cudaFree(s->dC);
    cudaFree(s->dD);
    cudaFree(s->dW);
    delete s;
}

int b200_session_gemm_host(b200_session *s, int dtype, const void *hA, const void *hBt, const float *hC, float *hD,
                           float alpha, float beta, int64_t M, int64_t N, int64_t K, const b200_gemm_params *p) {
    if (!s || !hA || !hBt || !hD) return B200_INVALID_POINTER;
    if (M > s->max_m || N > s->max_n || K > s->max_k) return B200_INVALID_SHAPE;
    if (beta != 0.0f && !hC) return B200_INVALID_POINTER;
    // Three streams: upload, launches, download. A and B^T go up in up to eight row blocks each, alternately
    // (A_0, B_0, A_1, B_1, ...). When A_t has landed, the band of D it completes - rows of A_t against the B^T
    // blocks before it - is multiplied as one GEMM and downloaded; when B_t has landed, the band of its columns
    // against all rows of A so far. What is computable grows with the square of what has been uploaded, so the
    // download stream starts early and ends one band after the last upload; both directions of the link are busy
    // for most of the call (two 256 MiB copies at once take 5.4 ms on the measured host, one 4.8 ms). Every band
    // is its own launch with its own tiling (the defaults of its shape unless the caller passed tunables), so the
    // result equals one launch over the whole problem up to the fp32 summation order inside a tile.
    const b200_gemm_params *const user_p = p;
    auto block_of = [](int64_t extent, int64_t granule) {
        const int parts = extent >= 8 * 2 * granule ? 8 : 4;   // sixteen measured slower (8.08 against 7.47 - 7.66 ms at 8192^3), four equal
        int64_t b = ((extent + parts - 1) / parts + granule - 1) / granule * granule;
        if (b < 2 * granule) b = 2 * granule;
        return b;
    };
    const int64_t gran_m = (user_p && user_p->tile_m > 0) ? user_p->tile_m : 256;
    const int64_t gran_n = (user_p && user_p->tile_n > 0) ? user_p->tile_n : 256;
    const int64_t brows = block_of(M, gran_m), bcols = block_of(N, gran_n);
    const int R = static_cast<int>((M + brows - 1) / brows), Cn = static_cast<int>((N + bcols - 1) / bcols);
    const char *hA8 = static_cast<const char *>(hA), *hB8 = static_cast<const char *>(hBt);
    char *dA8 = static_cast<char *>(s->dA), *dB8 = static_cast<char *>(s->dB);
    cudaError_t e = cudaSuccess;
    const int steps = R > Cn ? R : Cn;
    // An error return must not leave copies or kernels of this call in flight on the session's
    // streams: the caller may free or reuse its host buffers as soon as the call is back.
    auto drained = [s](int status) {
        cudaStreamSynchronize(s->stream);
        cudaStreamSynchronize(s->compute);
        cudaStreamSynchronize(s->download);
        return status;
    };
    // one band of D: rows [r0, r0 + rows) x columns [c0, c0 + cols), after the upload event `landed`
    auto band = [&](cudaEvent_t landed, cudaEvent_t computed, int64_t r0, int64_t rows, int64_t c0, int64_t cols) -> int {
        cudaError_t be = cudaEventRecord(landed, s->stream);
        if (be == cudaSuccess) be = cudaStreamWaitEvent(s->compute, landed, 0);
        if (be != cudaSuccess) return fail_cuda(be);
        if (rows <= 0 || cols <= 0) return B200_OK;
        b200_gemm_params local;
        const b200_gemm_params *bp = user_p;
        if (!bp) {
            default_params(rows, cols, K, &local, true, beta == 0.0f);   // as a call without tunables picks them
            bp = &local;
        }
        const size_t off = static_cast<size_t>(r0) * N + c0;
        const int st = gemm_impl(dtype, dA8 + static_cast<size_t>(r0) * K * 2, dB8 + static_cast<size_t>(c0) * K * 2,
                                 beta != 0.0f ? s->dC + off : nullptr, s->dD + off, alpha, beta, rows, cols, K, bp, s->dW, s->w_bytes,
                                 s->compute, nullptr, N);
        if (st != B200_OK) return st;
        be = cudaEventRecord(computed, s->compute);
        if (be == cudaSuccess) be = cudaStreamWaitEvent(s->download, computed, 0);
        if (be == cudaSuccess)
            be = cudaMemcpy2DAsync(hD + off, static_cast<size_t>(N) * 4, s->dD + off, static_cast<size_t>(N) * 4,
                                   static_cast<size_t>(cols) * 4, static_cast<size_t>(rows), cudaMemcpyDeviceToHost, s->download);
        return be == cudaSuccess ? B200_OK : fail_cuda(be);
    };
    for (int t = 0; t < steps; ++t) {
        if (t < R) {
            const int64_t r0 = t * brows, rows = (M - r0 < brows) ? (M - r0) : brows;
            e = cudaMemcpyAsync(dA8 + static_cast<size_t>(r0) * K * 2, hA8 + static_cast<size_t>(r0) * K * 2,
                                static_cast<size_t>(rows) * K * 2, cudaMemcpyHostToDevice, s->stream);
            if (e == cudaSuccess && beta != 0.0f)
                e = cudaMemcpyAsync(s->dC + static_cast<size_t>(r0) * N, hC + static_cast<size_t>(r0) * N,
                                    static_cast<size_t>(rows) * N * 4, cudaMemcpyHostToDevice, s->stream);
            if (e != cudaSuccess) return drained(fail_cuda(e));
            // rows of A_t against the B^T blocks 0 .. t-1 (all of them once B^T is complete)
            const int64_t have_cols = (t < Cn ? t : Cn) * bcols;
            const int st = band(s->up[2 * t], s->done[2 * t], r0, rows, 0, have_cols < N ? have_cols : N);
            if (st != B200_OK) return drained(st);
        }
        if (t < Cn) {
            const int64_t c0 = t * bcols, cols = (N - c0 < bcols) ? (N - c0) : bcols;
            e = cudaMemcpyAsync(dB8 + static_cast<size_t>(c0) * K * 2, hB8 + static_cast<size_t>(c0) * K * 2,
                                static_cast<size_t>(cols) * K * 2, cudaMemcpyHostToDevice, s->stream);
            if (e != cudaSuccess) return drained(fail_cuda(e));
            // columns of B_t against the rows of A_0 .. A_t (all of them once A is complete)
            const int64_t have_rows = (t + 1 < R ? t + 1 : R) * brows;
            const int st = band(s->up[2 * t + 1], s->done[2 * t + 1], 0, have_rows < M ? have_rows : M, c0, cols);
            if (st != B200_OK) return drained(st);
        }
    }
    e = cudaStreamSynchronize(s->download);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s->stream);
    if (e != cudaSuccess) return drained(fail_cuda(e));
    return B200_OK;
}

int b200_session_buffers(b200_session *s, void **dA, void **dBt, void **dC, void **dD) {
    if (!s) return B200_INVALID_POINTER;
    if (dA) *dA = s->dA;
    if (dBt) *dBt = s->dB;
    if (dC) *dC = s->dC;
    if (dD) *dD = s->dD;
    return B200_OK;
}

int b200_session_gemm_host_sharded(b200_session *s, int dtype, const void *hA_rows, const void *hBt_rows, const float *hC_rows,
                                   float *hD_rows, float alpha, float beta, int64_t m_rows, int64_t N, int64_t K, int world,
                                   int rank, void *const *peer_bt, void *const *peer_flags, int epoch,
                                   const b200_gemm_params *p) {
    if (!s || !hA_rows || !hBt_rows || !hD_rows || !peer_bt || !peer_flags) return B200_INVALID_POINTER;
    if (world < 1 || world > 8 || rank < 0 || rank >= world || epoch < 1) return B200_INVALID_CONFIG;
    if (m_rows <= 0 || m_rows > s->max_m || N > s->max_n || K > s->max_k || N <= 0 || K <= 0) return B200_INVALID_SHAPE;
    if (N % world || (N / world) % 256) return B200_INVALID_SHAPE;   // column blocks end on tile edges of every tile shape
    if (beta != 0.0f && !hC_rows) return B200_INVALID_POINTER;
    for (int o = 0; o < world; ++o)
        if (!peer_bt[o] || !peer_flags[o]) return B200_INVALID_POINTER;
    if (peer_bt[rank] != s->dB) return B200_INVALID_POINTER;         // this rank's entry is the session's own B^T buffer
    b200_gemm_params local;
    const int64_t cols = N / world;                       // B^T rows (= columns of D) per rank
    int64_t brows = ((m_rows + 3) / 4 + 255) / 256 * 256; // A is uploaded and multiplied in up to four row blocks
    if (brows > m_rows) brows = m_rows;
    const int R = static_cast<int>((m_rows + brows - 1) / brows);
    if (!p) {
        default_params(brows, cols, K, &local, true, beta == 0.0f);   // the shape of one block product
        p = &local;
    }
    const size_t slice_bytes = static_cast<size_t>(cols) * K * 2;
    const long long budget = static_cast<long long>(g_wait_budget_ns.load() * 2ull);
    int *const my_flags = static_cast<int *>(peer_flags[rank]);
    char *const dB8 = static_cast<char *>(s->dB);
    cudaError_t e = cudaSuccess;
    auto drained = [s](int status) {
        cudaStreamSynchronize(s->stream);
        cudaStreamSynchronize(s->push);
        cudaStreamSynchronize(s->compute);
        cudaStreamSynchronize(s->download);
        return status;
    };
    auto check = [&](int launch_error) { return launch_error == 0 ? cudaSuccess : static_cast<cudaError_t>(launch_error); };

    // upload stream: this rank's B^T rows first (every other GPU waits for them), then its A rows in up to four row
    // blocks (and the matching C rows), so that the first products and their downloads start while later rows are
    // still on their way up: the two copy directions run on different engines
    e = cudaMemcpyAsync(dB8 + static_cast<size_t>(rank) * slice_bytes, hBt_rows, slice_bytes, cudaMemcpyHostToDevice, s->stream);
    if (e == cudaSuccess) e = cudaEventRecord(s->b_ready, s->stream);
    if (e == cudaSuccess) e = check(launch_flag_set(my_flags + rank, epoch, s->stream));
    for (int i = 0; i < R && e == cudaSuccess; ++i) {
        const int64_t r0 = i * brows, rows = (m_rows - r0 < brows) ? (m_rows - r0) : brows;
        e = cudaMemcpyAsync(static_cast<char *>(s->dA) + static_cast<size_t>(r0) * K * 2,
                            static_cast<const char *>(hA_rows) + static_cast<size_t>(r0) * K * 2, static_cast<size_t>(rows) * K * 2,
                            cudaMemcpyHostToDevice, s->stream);
        if (e == cudaSuccess && beta != 0.0f)
            e = cudaMemcpyAsync(s->dC + static_cast<size_t>(r0) * N, hC_rows + static_cast<size_t>(r0) * N,
                                static_cast<size_t>(rows) * N * 4, cudaMemcpyHostToDevice, s->stream);
        if (e == cudaSuccess) e = cudaEventRecord(s->up[i], s->stream);
    }
    if (e != cudaSuccess) return drained(fail_cuda(e));

    // push stream: the rows just uploaded go to every other GPU over NVLink (one copy per peer, nearest rank first),
    // each followed by that peer's "rows of `rank` have arrived" flag. A peer's buffer is overwritten only after
    // that peer has announced the end of its previous product (its "done" flag here).
    e = cudaStreamWaitEvent(s->push, s->b_ready, 0);
    for (int d = 1; d < world && e == cudaSuccess; ++d) {
        const int o = (rank + d) % world;
        e = check(launch_flag_wait(my_flags + world + o, epoch - 1, budget, 900 + o, s->push));
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(static_cast<char *>(peer_bt[o]) + static_cast<size_t>(rank) * slice_bytes,
                                dB8 + static_cast<size_t>(rank) * slice_bytes, slice_bytes, cudaMemcpyDefault, s->push);
        if (e == cudaSuccess) e = check(launch_flag_set(static_cast<int *>(peer_flags[o]) + rank, epoch, s->push));
    }
    if (e != cudaSuccess) return drained(fail_cuda(e));

    // compute stream: column block by column block, own block first, each as soon as its B^T rows are here, and
    // within a column block one product per row block of A; download stream: every finished block of D goes back
    // while the next one is computed
    int n_done = 0;
    for (int d = 0; d < world && e == cudaSuccess; ++d) {
        const int j = (rank + d) % world;
        e = check(launch_flag_wait(my_flags + j, epoch, budget, 910 + j, s->compute));
        for (int i = 0; i < R && e == cudaSuccess; ++i) {
            const int64_t r0 = i * brows, rows = (m_rows - r0 < brows) ? (m_rows - r0) : brows;
            if (d == 0) e = cudaStreamWaitEvent(s->compute, s->up[i], 0);
            if (e != cudaSuccess) break;
            const size_t off = static_cast<size_t>(r0) * N + static_cast<size_t>(j) * cols;
            const int st = gemm_impl(dtype, static_cast<char *>(s->dA) + static_cast<size_t>(r0) * K * 2,
                                     dB8 + static_cast<size_t>(j) * slice_bytes, beta != 0.0f ? s->dC + off : nullptr, s->dD + off,
                                     alpha, beta, rows, cols, K, p, s->dW, s->w_bytes, s->compute, nullptr, N);
            if (st != B200_OK) return drained(st);
            cudaEvent_t ev = s->done[n_done++ % 16];     // recorded and waited for at once: safe to record again later
            e = cudaEventRecord(ev, s->compute);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(s->download, ev, 0);
            if (e == cudaSuccess)
                e = cudaMemcpy2DAsync(hD_rows + off, static_cast<size_t>(N) * 4, s->dD + off, static_cast<size_t>(N) * 4,
                                      static_cast<size_t>(cols) * 4, static_cast<size_t>(rows), cudaMemcpyDeviceToHost, s->download);
        }
    }
    // tell every GPU that this one no longer reads the B^T rows of this epoch
    for (int o = 0; o < world && e == cudaSuccess; ++o)
        if (o != rank) e = check(launch_flag_set(static_cast<int *>(peer_flags[o]) + world + rank, epoch, s->compute));
    if (e != cudaSuccess) return drained(fail_cuda(e));
    e = cudaStreamSynchronize(s->download);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s->compute);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s->push);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s->stream);
    if (e != cudaSuccess) return drained(fail_cuda(e));
    return B200_OK;
}

int b200_device_status(void *stream, int info[4]) {
    int rec[4] = {0, 0, 0, 0};
    const int e = read_device_status(rec, static_cast<cudaStream_t>(stream));
    if (e != 0) return fail_cuda(static_cast<cudaError_t>(e));
    if (info)
        for (int i = 0; i < 4; ++i) info[i] = rec[i];
    return rec[0] == 0 ? B200_OK : rec[0];
}

void b200_set_wait_budget_ns(uint64_t ns) { g_wait_budget_ns.store(ns ? ns : 1); }

void b200_set_profile_buffer(void *device_ptr, int blocks) {
    g_prof_ptr.store(static_cast<long long *>(device_ptr));
    g_prof_blocks.store(device_ptr ? blocks : 0);
}

int b200_profile_slots(void) { return profile_slots(); }

const char *b200_status_string(int status) {
    switch (status) {
        case B200_OK: return "ok";
        case B200_INVALID_CONFIG: return "invalid configuration (tunables outside the domain or over the shared/tensor memory budget)";
        case B200_INVALID_SHAPE: return "invalid shape (M, N, K must be positive, N a multiple of 4 and K of 8; split-K and multi-GPU forms add their own rules)";
        case B200_INVALID_POINTER: return "null or misaligned pointer";
        case B200_CUDA_ERROR: return "CUDA error";
        case B200_DEVICE_TIMEOUT: return "a bounded wait inside the kernel expired";
        case B200_WORKSPACE_TOO_SMALL: return "workspace missing or too small";
        case B200_UNSUPPORTED_DEVICE: return "no sm_100 device: this library has no other code path";
        default: return "unknown status";
    }
}

int b200_last_cuda_error(void) { return t_last_cuda_error; }

int b200_num_sms(void) {
    const DeviceInfo *dev = nullptr;
    if (device_info(&dev) != B200_OK) return -1;
    return dev->num_sms;
}

int b200_fill_u16_device(void *dst, int64_t begin, int64_t count, uint64_t seed, uint64_t tensor_id, int dist,
                         float sigma, int dtype, void *stream) {
    if (!dst || count < 0) return B200_INVALID_POINTER;
    if (count == 0) return B200_OK;
    int blocks = static_cast<int>((count + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    fill_u16_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint16_t *>(dst), begin, count,
                                                                           synth::key_of(seed, tensor_id), dist, sigma, dtype);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? B200_OK : fail_cuda(e);
}

int b200_fill_f32_device(float *dst, int64_t begin, int64_t count, uint64_t seed, uint64_t tensor_id, int dist,
                         float sigma, void *stream) {
    if (!dst || count < 0) return B200_INVALID_POINTER;
    if (count == 0) return B200_OK;
    int blocks = static_cast<int>((count + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    fill_f32_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(dst, begin, count, synth::key_of(seed, tensor_id),
                                                                           dist, sigma);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? B200_OK : fail_cuda(e);
}

void b200_fill_u16_host(uint16_t *dst, int64_t begin, int64_t count, uint64_t seed, uint64_t tensor_id, int dist,
                        float sigma, int dtype) {
    const uint64_t key = synth::key_of(seed, tensor_id);
    for (int64_t i = 0; i < count; ++i) dst[i] = synth::value_u16(key, static_cast<uint64_t>(begin + i), dist, sigma, dtype);
}

void b200_fill_f32_host(float *dst, int64_t begin, int64_t count, uint64_t seed, uint64_t tensor_id, int dist,
                        float sigma) {
    const uint64_t key = synth::key_of(seed, tensor_id);
    for (int64_t i = 0; i < count; ++i) dst[i] = synth::value(key, static_cast<uint64_t>(begin + i), dist, sigma);
}

}  // extern "C"
