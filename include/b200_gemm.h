/*
 * b200_gemm.h - C ABI of the B200 (sm_100a) asynchronous tensor-core GEMM.
 *
 *     D = alpha * A * B^T + beta * C
 *
 * A is m x k row-major, Bt is B stored transposed as n x k row-major (both fp16 or both bf16),
 * C and D are m x n row-major fp32, accumulation is fp32. Every pointer of the device entry
 * points is a DEVICE pointer owned by the caller; the calls allocate nothing, enqueue on the
 * given stream and return without synchronising.
 *
 * Each entry point names the interface of the reference (alfin3/cuda-kernel-opt) it stands in
 * for, as file:line of that project.
 */
#ifndef B200_GEMM_H
#define B200_GEMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes. The reference's launchers return void, assert on the parameter domain and check
 * CUDA errors only under -DDEBUG (matmul_shmem_tc_async.cu:45-54, :511-517); here every failure
 * is a return value and nothing asserts, aborts or traps. */
enum {
    B200_OK = 0,
    B200_INVALID_CONFIG = 1,   /* tunables outside the supported domain, or over the smem/TMEM budget */
    B200_INVALID_SHAPE = 2,    /* M, N, K not positive, N not a multiple of 4 or K not a multiple of 8 (rows must be
                                  16-byte multiples); the split-K and multi-GPU forms add their own rules. Ragged
                                  tile edges are accepted here; the reference-shaped launchers of b200_matmul.h
                                  keep the reference's tile-multiple rule */
    B200_INVALID_POINTER = 3,  /* null or misaligned operand (A, Bt, D need 16-byte alignment) */
    B200_CUDA_ERROR = 4,       /* a CUDA runtime/driver call failed; see b200_last_cuda_error() */
    B200_DEVICE_TIMEOUT = 5,   /* a bounded wait inside the kernel expired; see b200_device_status() */
    B200_WORKSPACE_TOO_SMALL = 6,
    B200_UNSUPPORTED_DEVICE = 7 /* not an sm_100 GPU */
};

enum { B200_F16 = 0, B200_BF16 = 1 };

/* Tunables. The first twelve are the reference launcher's own (matmul_shmem_tc_async_opt_port_2.cu
 * :1088-1109); tile_dim is split into tile_m/tile_n and cta_group/split_k are added for the B200.
 *
 * tile_m             output-tile rows: 128 (one CTA), 256 (two-CTA pair, cta_group = 2) or 64; 512 with
 *                    cta_group = 2 is the tall pair: each CTA stages 256 rows of A and issues them as two
 *                    128-row MMA atoms against one B^T stage (a quarter fewer operand bytes per flop); its
 *                    two accumulators fill the tensor memory at tile_n = 256, so a tile's drain is not hidden
 *                    behind the next tile's MMAs. Whole tiles only (split_k = 1, no tail split, no swap),
 *                    bar_step_rows_a = 512
 * tile_n             output-tile columns: multiple of 16 in [16, 256]
 * segment_dim_k      K extent staged per pipeline stage; multiple of 64
 * bar_steps_a/b      number of leading sub-tiles of the A / B^T stage buffer with a private "full"
 *                    barrier; the rest share one residual barrier (port_2.cu:627-630)
 * bar_step_rows_a/b  rows of A / rows of B^T (= columns of the tile) per sub-tile; equal to the
 *                    tile extent = no sub-tiles = shift synchronisation off (port_1.cu:508-509). Every B^T
 *                    sub-tile has its own MMAs, issued as it lands. A one-CTA 128 x (<= 128) tile with
 *                    bar_step_rows_a <= 64 is issued as two 64-row MMA atoms, the upper one as soon as the
 *                    barriers of rows 0-63 are complete (the reference's per-fragment-row start,
 *                    port_1.cu:406-433); in every other form the A steps set the copy granularity only
 * tile_group_m       tile rows per L2 rasterisation group (port_0.cu:201-210)
 * num_stages         depth of the shared-memory ring
 * num_producer_warps 1 = one warp issues the A and the B^T copies; >= 2 = separate A and B^T
 *                    issuing warps (the reference's split, port_1.cu:197); further warps idle
 * num_consumer_warps 4 or 8 warps draining the accumulator (one or two per 32 TMEM lanes)
 * num_sms            size of the persistent grid (CTAs); 0 = all SMs of the device
 * cta_group          1, or 2 for the two-CTA tcgen05 pair (tile_m = 256 or 512)
 * split_k            K slices computed by different CTAs into the workspace and summed; 1 = off
 * epilogue, l2_hint  see the fields
 */
typedef struct b200_gemm_params {
    int tile_m;
    int tile_n;
    int segment_dim_k;
    int bar_steps_a;
    int bar_steps_b;
    int bar_step_rows_a;
    int bar_step_rows_b;
    int tile_group_m;
    int num_stages;
    int num_producer_warps;
    int num_consumer_warps;
    int num_sms;
    int cta_group;
    int split_k;
    int epilogue;  /* 0 = registers -> global 128-bit stores, 1 = registers -> smem -> TMA store */
    int l2_hint;   /* L2 eviction priority of the operand loads: 0 = normal for both, 1 = A evict_last and
                      B^T evict_first (A row panels are the reused operand of the grouped tile order),
                      2 = A evict_last, 3 = both evict_last */
    int diagnostic; /* must be 0. Bit 0 issues no MMA, bit 1 no operand load: pipeline ceilings for
                       profiling; the output is garbage. Bits 2 and 3 (with cluster_reduce) withhold the
                       "slice staged" / "slice read" arrivals between the CTAs of a cluster, so those
                       bounded waits expire: the launch returns normally with a B200_DEVICE_TIMEOUT
                       record (barrier ids 701 / 700) and an unfinished D; bit 4 (with tail_split) withholds the
                       "partial stored" flags of its fix-up in the same way (wait ids 800 + warp);
                       for tests of those paths. Bit 5 stores D with normal L2 priority where the library would
                       mark its lines evict_first (TMA-store epilogue, D of 64 MiB or more): an A/B switch */
    int k_order;    /* 0 = every tile sums K ascending; 1 = serpentine: every other tile of a CTA walks K downwards,
                       so consecutive waves meet their shared operand panels while they are still in L2.
                       Changes the fp32 summation order of those tiles (not the tolerance) */
    int tail_split; /* 1 = the tiles that do not fill a wave of the persistent grid (T tiles on S CTAs or CTA pairs
                       leave r = T mod S for a last, partly idle wave) are cut into s equal K slices each; the
                       r * s slice units run first, dealt to the CTAs in rounds, slice-major, so that CTAs
                       running together stay in step along K and share operand panels in L2; the tail then
                       costs ceil(r * s / S) / s tile times instead of one (s <= 8 is chosen by that cost; off
                       when under 2 % of the launch would be gained). A cut tile is finished inside the kernel
                       by the CTA that runs its last slice, which adds the other slices' fp32 partials
                       (ascending K, deterministic) from the workspace before the usual alpha / beta / store:
                       no second kernel. Successor of the reference's persistent tile loop
                       (matmul_shmem_tc_async.cu:251-252), which leaves SMs idle in the last wave. Takes effect
                       only when the call is given b200_gemm_workspace_bytes of workspace; without it the plain
                       schedule runs. At most 16 such launches may be in flight on a device at once (they share
                       flag sets inside the library); launches on one stream never are. 0 = off */
    int swap_ab;    /* 1 = operand roles swapped inside the kernel for skinny M (decode shapes): the rows of B^T feed
                       the 64/128-row side of the MMA and the few rows of A its N side, so a stage holds
                       tile_n rows of weights and only tile_m rows of activations, and the accumulator is
                       written to D transposed (coalesced along N). Then tile_n is 64 or 128 with cta_group = 1,
                       or 256 with the two-CTA pair (cta_group = 2: each CTA stages 128 weight rows and half of
                       the activation rows); tile_m is a multiple of 16 (32 with the pair) in [16, 256]; the
                       bar_step fields follow their operands; needs tail_split = 0 and drains with plain
                       stores. Same results as 0 */
    int cluster_reduce; /* 1 (with swap_ab = 1, split_k 2, 4 or 8, tile_m <= 128, cta_group * split_k <= 8) = the
                       split_k slices of a tile run as the CTAs (or CTA pairs) of one thread-block cluster and
                       are summed through distributed shared memory, in slice order: no workspace, no second
                       kernel, same bits as the workspace form. 0 = slices meet in the workspace */
    int overlap_launch; /* 1 = programmatic dependent launch: the kernel is launched with programmatic stream
                       serialisation, runs its set-up (barriers, tensor memory, descriptor prefetch) while the
                       previous kernel of the stream finishes, waits for that kernel (griddepcontrol.wait)
                       before its first global access, and lets the next such launch start early in the same
                       way. Results and ordering are those of a normal launch; for chains of short GEMMs
                       (decode steps), where launch gaps are a visible share of a step. 0 = normal launch */
} b200_gemm_params;

/* Fills *p with the tuned default for the shape (what the reference's harness hard-codes per
 * sweep, port_2.cu:1518-1564). dtype is B200_F16 or B200_BF16. Tuned for alpha * A * B^T with beta = 0 and
 * fp32 D: for 8192^3-sized squares and their row shards that is the tall pair (tile_m = 512), whose exposed
 * drain is slower with C to read; a call with p = NULL knows beta and the output type and keeps the 256-row
 * pair for beta != 0, fp16 output and b200_gemm_push. */
int b200_gemm_default_params(int64_t M, int64_t N, int64_t K, int dtype, b200_gemm_params *p);
/* The same without the swapped forms (swap_ab = 0): the tuned plain tile for the shape, the starting point
 * for callers that set tile_m / tile_n / epilogue themselves in the reference's meaning. */
int b200_gemm_default_params_plain(int64_t M, int64_t N, int64_t K, int dtype, b200_gemm_params *p);
/* The defaults a call with p = NULL would take, given what such a call knows beyond the shape: beta and
 * whether C and D are fp16 (b200_gemm_f16_out_f16). No reference counterpart. */
int b200_gemm_default_params_for_call(int64_t M, int64_t N, int64_t K, int dtype, float beta, int fp16_out, b200_gemm_params *p);

/* Host-only validation: the reference's asserts (port_2.cu:1112-1123) and its harness's
 * shared-memory filter (port_2.cu:1229-1232) as a status. Touches no GPU. */
int b200_gemm_validate(int64_t M, int64_t N, int64_t K, int dtype, const b200_gemm_params *p);

/* Dynamic shared memory the configuration needs, in bytes; the counterpart of get_shmem_req
 * (port_2.cu:1057-1086). Negative if the configuration is invalid. */
int64_t b200_gemm_smem_bytes(int dtype, const b200_gemm_params *p);

/* Bytes of caller-provided device workspace for the configuration: what split_k > 1 (without
 * cluster_reduce) needs, or what tail_split = 1 can use on this shape (0 when nothing would be cut);
 * 0 otherwise. With num_sms = 0 the grid follows the current device (148 SMs assumed
 * when there is none). */
int64_t b200_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, const b200_gemm_params *p);

/* Lists the work units CTA group `group` (a CTA, or a two-CTA pair) of a launch on num_sms SMs walks, in
 * order: units[6*i .. 6*i+5] = {first row, first column of the tile (of the transposed problem with
 * swap_ab), first K segment, end K segment, kind, K slice}; kind 0 = the CTA finishes the tile alone,
 * 1 = the last K slice of a cut tile: the CTA finishes the tile with the other slices' partials (tail_split),
 * 2 = an earlier K slice, whose partial the finishing CTA adds. Host arithmetic only, the same code the kernel runs:
 * for tests and tuners (in the reference the schedule is the loop `for (tile = blockIdx.x; tile < tiles;
 * tile += gridDim.x)`, matmul_shmem_tc_async.cu:251-252). Returns the number of units (which may exceed
 * max_units; only that many are written), -1 for an invalid configuration or group; *num_groups_out
 * (may be null) receives the number of groups. */
int b200_gemm_schedule(int64_t M, int64_t N, int64_t K, const b200_gemm_params *p, int num_sms, int group, int *units,
                       int max_units, int *num_groups_out);

/* The GEMM. Stands in for gemm_shmem_tc_async (matmul_shmem_tc_async.cu:494-557) and
 * gemm_shmem_tc_async_opt_port (matmul_shmem_tc_async_opt_port_0.cu:515-579, _1.cu:889-965,
 * _2.cu:1088-1168) with DT = half (b200_gemm_f16) or bf16 (b200_gemm_bf16) and DT_ACC = float.
 * C may be null when beta == 0. workspace may be null when none is needed. stream is a
 * cudaStream_t (null = the legacy default stream, which is what the reference launches on). */
int b200_gemm_f16(const void *A, const void *Bt, const float *C, float *D, float alpha, float beta, int64_t M,
                  int64_t N, int64_t K, const b200_gemm_params *p, void *workspace, size_t workspace_bytes,
                  void *stream);
int b200_gemm_bf16(const void *A, const void *Bt, const float *C, float *D, float alpha, float beta, int64_t M,
                   int64_t N, int64_t K, const b200_gemm_params *p, void *workspace, size_t workspace_bytes,
                   void *stream);

/* The same product with fp16 C and D (m x n row-major halves): stands in for the reference's DT = DT_ACC = half
 * instances of the launchers above (matmul_shmem_tc_async.cu:411-478 instantiate both). Accumulation stays
 * fp32 in tensor memory and the result is rounded to fp16 once (the reference's half instances accumulate in
 * half), so it is at least as close to the exact product. Needs no workspace (tail_split does not engage
 * without one): configurations whose K slices meet in a workspace (split_k > 1
 * without cluster_reduce) are B200_INVALID_CONFIG here. */
int b200_gemm_f16_out_f16(const void *A, const void *Bt, const void *C, void *D, float alpha, float beta, int64_t M,
                          int64_t N, int64_t K, const b200_gemm_params *p, void *stream);

/* Split-K GEMM that allocates nothing and needs no workspace from the caller. It has no
 * counterpart in the reference (whose launchers never split K and never need scratch memory).
 *
 * For callers that cannot allocate device memory or be handed any: a step of a serving loop
 * that must not hit cudaMalloc's device synchronisation, a callback that runs while another
 * library holds its allocator lock, a plugin host that passes fixed input and output buffers only.
 * The per-slice fp32 partial products go to a 32 MiB device array built into the library (every
 * GPU that loads the library holds it until the process exits), so split_k * M * N must not
 * exceed 8 Mi values; larger problems return B200_WORKSPACE_TOO_SMALL and belong to
 * b200_gemm_f16 / b200_gemm_bf16 with a caller workspace. p->split_k must be >= 2.
 *
 * The first call on a device looks up the array's device address (once per device). With lazy
 * module loading that look-up is also the moment the driver loads this part of the library and
 * places the 32 MiB array in device memory, which can stall the device: make the first call at
 * start-up, outside any stream capture and outside the latency-critical region. No cudaMalloc,
 * cudaFree or allocating library routine is called, on the first call or later, and from the second
 * call on the device's free memory does not change. All calls on a device share the one array: it keeps the
 * previous call's partials, every element a call reads it has written first (nothing needs
 * clearing), and two calls whose kernels overlap on the GPU (different streams, no ordering)
 * race on it - order them. dtype is B200_F16 or B200_BF16; other arguments as b200_gemm_f16. */
int b200_gemm_splitk_noalloc(int dtype, const void *A, const void *Bt, const float *C, float *D, float alpha, float beta,
                             int64_t M, int64_t N, int64_t K, const b200_gemm_params *p, void *stream);

/* Split-K across the GPUs of a box with the reduce-scatter fused into the GEMM epilogue. The
 * reference is single-GPU (cudaSetDevice(0), matmul_shmem_tc_async_opt_port_2.cu:1503-1510) and
 * never splits K; this is the multi-GPU form of the same launcher for tall-K problems.
 *
 * Rank r multiplies its K slice (A: M x K_local, Bt: N x K_local). GPU o owns rows
 * [o*M/world, (o+1)*M/world) of D. b200_gemm_push stores every finished fp32 tile straight into
 * the owner's slot area over NVLink (plain peer stores, no TMA on remote memory): slot_ptrs[o]
 * is owner o's area of world x (M/world) x N floats, indexed [source rank][row][col], as mapped
 * into this process (b200_peer_import); flag_ptrs[o] is owner o's array of `world` ints. The last
 * CTA to finish writes `epoch` into flag[o][rank] on every owner. done_counter is a zeroed
 * local unsigned int. M/world must be a multiple of 128 (256 for the two-CTA tile). With
 * p->split_k > 1 the K slices of this GPU are first summed from the caller's workspace
 * (b200_gemm_workspace_bytes) and the sum is what travels, as coalesced 128-bit peer stores.
 *
 * b200_push_reduce, enqueued on the owner after its own b200_gemm_push, waits (bounded; a
 * DEVICE_TIMEOUT record if a peer never arrives) until all `world` flags have reached `epoch`
 * (a flag already past it also counts: with two slot areas a fast peer may have pushed its next
 * step before this owner looks), then
 * writes D_rows = alpha * sum over sources of slot[src] + beta * C_rows, sources in ascending
 * order. Use a new epoch (> 0, increasing) for every GEMM; slots of epoch e may be overwritten
 * only after every rank has finished b200_push_reduce of epoch e (a barrier per step, or two
 * alternating slot areas). After a DEVICE_TIMEOUT read the record with b200_device_status before
 * the next push: while a record is pending a push raises no flags. Swapped roles and the tall pair
 * (tile_m = 512, which b200_gemm_default_params returns for large squares) are refused with
 * B200_INVALID_CONFIG: pass p = NULL for the defaults of this call, or set tile_m = 256. */
int b200_gemm_push(int dtype, const void *A, const void *Bt, int64_t M, int64_t N, int64_t K, const b200_gemm_params *p,
                   int world, int rank, void *const *slot_ptrs, void *const *flag_ptrs, void *done_counter, int epoch,
                   void *workspace, size_t workspace_bytes, void *stream);
int b200_push_reduce(const float *my_slots, const int *my_flags, int world, int epoch, const float *C, float *D, float alpha,
                     float beta, int64_t rows, int64_t N, void *stream);
/* Device memory that other processes of the box can map (cudaMalloc + CUDA IPC), zero-filled; the
 * 64-byte handle travels by any host channel (the bench uses torch.distributed). */
int b200_peer_alloc(size_t bytes, void **out);
int b200_peer_free(void *ptr);
int b200_peer_export(void *ptr, unsigned char handle[64]);
int b200_peer_import(const unsigned char handle[64], void **out);
int b200_peer_release(void *imported);

/* Host-buffer call: what the reference's harness does around one launch - cudaMemcpy of A, B^T
 * (and C when beta != 0) to the device, the launch, cudaMemcpy of D back, which is also the
 * synchronisation (port_2.cu:1210-1212, :1238-1242). Device buffers come from a session created
 * once at the maximal dimensions, as the harness cudaMallocs once (port_2.cu:1200-1203). Host
 * pointers may be pageable or pinned (with pinned memory A and B^T go up in up to eight row blocks each and the
 * band of D every block completes is multiplied and downloaded while later uploads run, three streams; every band is
 * its own launch, so the result equals one launch over the whole problem up to fp32 summation order). Returns after
 * D is in host memory. */
typedef struct b200_session b200_session;
int b200_session_create(int64_t max_m, int64_t max_n, int64_t max_k, b200_session **out);
void b200_session_destroy(b200_session *s);
int b200_session_gemm_host(b200_session *s, int dtype, const void *hA, const void *hBt, const float *hC, float *hD,
                           float alpha, float beta, int64_t M, int64_t N, int64_t K, const b200_gemm_params *p);

/* The host-buffer call on the GPUs of one box, one process and one session per GPU, for D = A * B^T with the rows
 * of A and D split over the ranks and B^T needed whole on every GPU (the M-shard of a square problem). The
 * reference's harness is single-GPU (cudaSetDevice(0), matmul_shmem_tc_async_opt_port_2.cu:1503-1510); done naively,
 * every rank would upload all of B^T over its own PCIe link. Here B^T crosses PCIe once: rank r uploads only rows
 * [r*N/world, (r+1)*N/world) of B^T (hBt_rows) and its own rows of A (hA_rows, m_rows x K), copies its B^T rows
 * into the other GPUs' B^T buffers over NVLink (plain peer copies, one per peer), and multiplies column block by
 * column block as the blocks arrive, own block first, downloading each finished block of D (hD_rows, m_rows x N)
 * while the next is computed. peer_bt[o] is rank o's session B^T buffer (b200_session_buffers) as mapped into this
 * process (b200_peer_export / b200_peer_import; peer_bt[rank] is this session's own), peer_flags[o] rank o's array
 * of 2 * world ints from b200_peer_alloc (zeroed): [src] = rows of src have arrived (epoch), [world + src] = src has
 * finished its product of that epoch, so its buffer may be overwritten. epoch = 1, 2, 3, ... per call, the same on
 * every rank. N / world must be a multiple of 256. Waits for peers are on the device and bounded (wait ids 900 + peer
 * and 910 + block in the DEVICE_TIMEOUT record). Returns when D's rows are in host memory. */
int b200_session_buffers(b200_session *s, void **dA, void **dBt, void **dC, void **dD);
int b200_session_gemm_host_sharded(b200_session *s, int dtype, const void *hA_rows, const void *hBt_rows, const float *hC_rows,
                                   float *hD_rows, float alpha, float beta, int64_t m_rows, int64_t N, int64_t K, int world,
                                   int rank, void *const *peer_bt, void *const *peer_flags, int epoch,
                                   const b200_gemm_params *p);

/* Synchronises the stream and reports whether any kernel of this library hit a bounded-wait
 * timeout on the current device since the last call. info (may be null) receives
 * {code, block, barrier id, phase}. Clears the record. Barrier ids of the GEMM kernel: 100 + stage a producer's
 * wait for a free stage, 300 + slot the MMA thread's wait for a drained accumulator (301 with the tall pair: the
 * lower atom's columns), 400 / 500 + stage its waits for operand data, 600 + slot a draining warp's wait for a
 * finished accumulator, 700 - 703 the cluster reduce, 800 + warp the tail split's fix-up. */
int b200_device_status(void *stream, int info[4]);
/* Test hook: the budget of every in-kernel wait, in nanoseconds (default 2e9). */
void b200_set_wait_budget_ns(uint64_t ns);

/* Tracing hook: when device_ptr is non-null, the first `blocks` CTAs of every later GEMM launch
 * write b200_profile_slots() int64 counters each (clock64 cycles) into it: [0..2] A-producer {cycles waiting for free
 * stages, cycles in loop, stages filled}, [3..5] the same for a separate B^T producer, [6..9] MMA
 * thread {cycles waiting for data, cycles waiting for a free accumulator, cycles in loop, stages},
 * [10..12] first epilogue warp {cycles waiting for a finished tile, cycles in loop, tiles}, [13..15] %globaltimer
 * (ns) at kernel entry, after set-up and at exit, [16..17] A-side shift synchronisation {pipeline stages whose first
 * MMAs were issued before the stage's last rows of A had landed, stages}. The reference only times whole launches
 * with CUDA events (matmul_shmem_tc_async.cu:787-795). */
void b200_set_profile_buffer(void *device_ptr, int blocks);
/* int64 slots per CTA in that buffer: 18. A diagnostic build of the library (-DB200_TIMELINE) has 34: there
 * [16..31] are %globaltimer stamps of set-up and role milestones (cuda-kernel-opt_b200/timeline.py prints them) and
 * the A-side shift pair sits at [32..33]. */
int b200_profile_slots(void);

const char *b200_status_string(int status);
int b200_last_cuda_error(void); /* cudaError_t of the last failed CUDA call on this thread */
int b200_num_sms(void);         /* multiprocessor count of the current device, <= 0 on error */

/* Seeded synthetic inputs: element `index` of tensor `tensor_id` under `seed` from a counter
 * hash, identical on host and device. dist 0 = uniform [-1, 1), 1 = normal(0, sigma) (sum of
 * twelve uniforms). The reference fills with rand() seeded from the clock (matmul_test.h:239,
 * :328-339), which cannot be reproduced; these replace it. */
int b200_fill_u16_device(void *dst, int64_t begin, int64_t count, uint64_t seed, uint64_t tensor_id, int dist,
                         float sigma, int dtype, void *stream);
int b200_fill_f32_device(float *dst, int64_t begin, int64_t count, uint64_t seed, uint64_t tensor_id, int dist,
                         float sigma, void *stream);
void b200_fill_u16_host(uint16_t *dst, int64_t begin, int64_t count, uint64_t seed, uint64_t tensor_id, int dist,
                        float sigma, int dtype);
void b200_fill_f32_host(float *dst, int64_t begin, int64_t count, uint64_t seed, uint64_t tensor_id, int dist,
                        float sigma);

#ifdef __cplusplus
}
#endif
#endif /* B200_GEMM_H */
