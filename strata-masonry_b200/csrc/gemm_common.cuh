// Shared between the kernels' translation units and the C-ABI layer: error plumbing,
// launch descriptors, the tile raster, tensor-map encoding.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

#include "../../include/strata_masonry_b200.h"

namespace smb {

// --------------------------------------------------------------------------- errors
// Record a message for smb_last_error() (thread-local) and return `code`.
int set_error(int code, const char* fmt, ...);
int set_cuda_error(cudaError_t e, const char* what);
// Text for a kernel's status word (ptx.cuh: DeviceStatus).
const char* device_status_name(int code);

// --------------------------------------------------------------------------- communicator (gather.cu)
// In-place NCCL all-gather of equal byte blocks: rank r's block already sits at
// buf + r * block_bytes; afterwards every rank holds all blocks.  Stream-ordered.
int comm_allgather_inplace(smb_comm* comm, void* buf, size_t block_bytes, cudaStream_t stream);
int comm_world(const smb_comm* comm);
int comm_rank(const smb_comm* comm);
int comm_device(const smb_comm* comm);

// --------------------------------------------------------------------------- self test
// One CTA waits `budget_cycles` on an mbarrier nobody arrives at and then records
// kDevTimeoutProbe in `status` (device memory); `waited_cycles` (device, optional) receives how
// long it waited.  Stream-ordered.  selftest.cu.
int wait_probe_launch(int* status, long long budget_cycles, long long* waited_cycles, cudaStream_t stream);

// --------------------------------------------------------------------------- raster
// Map a flat tile index onto (tile_m, tile_n).  Tiles are walked in groups of `group_m`
// tile rows; inside a group the M index runs fastest.  With ~74 clusters working on
// consecutive indices, one wave touches about group_m A panels and 74 / group_m B panels
// at the same K position, so both operands are shared through L2.  (The reference gets
// the same effect from its blocked raster, dense_gemm_nvfp4.cu:358-434.)
__host__ __device__ inline void tile_coords(int t, int tiles_m, int tiles_n, int group_m, int& tm,
                                            int& tn) {
  const int per_group = group_m * tiles_n;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int rows = (tiles_m - first_m) < group_m ? (tiles_m - first_m) : group_m;
  const int r = t - g * per_group;
  tm = first_m + r % rows;
  tn = r / rows;
}

// Default raster group height (tile rows walked M-fastest before the walk moves on along N).
// Two things pull on it.  A wave of ~74 clusters that spans g tile rows and 74 / g tile columns
// touches g A panels and 74 / g B panels, least for g around 8 to 12; and tiles of one row should
// run close together in time so that its A panel is still in L2.  Measured (sustained TFLOP/s):
//   BF16 8192^3 (256 x 512 tiles): g = 4 1320-1346, 8 1345-1370, 16 1330-1351, 32 1239-1287;
//   BF16 8192 x 8192 x 4096: 8 1600, 16 1614, 32 1572;  30720 x 2048 x 4096 (256 x 256 tiles): 8 1565,
//   16 1557, 32 1390;  14080 x 5120 x 2048: 8 1552, 16 1542, 32 1537.
// `row_bytes` = bytes of one row of A.  BF16: 32 MB of A per group, kept between 8 and 16 rows.
// `b_bytes` = size of the other operand: one that cannot stay in L2 between groups anyway (above
// 256 MB) is read from DRAM once per group, so the groups are made as tall as L2 has room for the
// A panel (16 rows at K = 8192: 64 MB).  32768 x 57344 x 8192, groups of 8 / 16 / 24 rows, sustained
// TFLOP/s: 1383-1392 / 1397-1417 / 1348-1349 (DRAM reads per launch at 8 rows with both operands
// marked evict-last: 58.5 GB, eleven times the operands).
inline int raster_group_rows(int tiles_m, long long row_bytes, long long b_bytes = 0) {
  long long rows = (32ll << 20) / (256 * (row_bytes > 0 ? row_bytes : 1));
  if (b_bytes > (256ll << 20)) rows = (64ll << 20) / (256 * (row_bytes > 0 ? row_bytes : 1));
  if (rows < 8) rows = 8;
  if (rows > 16) rows = 16;
  if (rows > tiles_m) rows = tiles_m;
  return static_cast<int>(rows);
}
// Block-scaled kernel (A is a quarter the size, and the tile list ends every group with narrower
// tiles): all rows in one group when they are fewer than the clusters and A as a whole stays in
// L2 (32 MB) - the narrow tiles then all come last, which also evens out the last wave - else 8.
// Measured (TFLOP/s, group of 4 / 8 / 16 / 32 / all rows): 8192^3 (32 rows) 6150 / 6007 / 6110 /
// 6200 / 6200;  14080 x 2048 x 4096 (55 rows) 5213 / 5217 / 5247 / 5293 / 5337;  14080 x 5120 x 2048
// 4700 / 4698 / 4635 / 4551 / 4672;  30720 x 2048 x 4096 (120 rows) 5352 / 5352 / 5363 / 5353 / 5250;
// 30720 x 5120 x 2048 4814 / 4782 / 4740 / 4662 / 4490;  30720 x 4096 x 8192 6230 / 6238 / 6145 / 6136 / -.
inline int raster_group_rows_fp4(int tiles_m, long long row_bytes) {
  const long long a_bytes = static_cast<long long>(tiles_m) * 256 * row_bytes;
  if (tiles_m <= 64 && a_bytes <= (32ll << 20)) return tiles_m;
  return tiles_m < 8 ? tiles_m : 8;
}

// --------------------------------------------------------------------------- tensor maps
// 2-D row-major tensor [rows, cols] of `elem_bytes`-wide elements, `ld_bytes` between rows,
// copied in boxes of [box_rows, box_cols].  `swizzle128`: 128-byte shared-memory swizzle
// (box_cols * elem_bytes must then be 128).  Out-of-range elements read as zero.
// Counterpart of make_tma_2d_tiled (reference src/primitives/23_tma_tensormap.cuh:43-64).
int encode_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                   uint64_t rows, uint64_t cols, uint64_t ld_bytes, uint32_t box_rows,
                   uint32_t box_cols, bool swizzle128);

// Extra destinations of every stored box of D (see epilogue.cuh): the all-gather of a
// column-sharded GEMM fused into the epilogue.
// Two uses.  Replicate (route_rows == 0): every stored box goes to D and to all `count` (<= 7)
// destinations, the all-gather of a column-sharded GEMM.  Route (route_rows > 0): D is not
// written; rows [b * route_rows, (b + 1) * route_rows) go to destination b only, at their row
// inside the block: the scatter half of a reduce-scatter after a K-sharded GEMM, every rank
// delivering the row block of its partial product that rank b owns.
constexpr int kMaxPeerCopies = 8;
struct PeerCopies {
  int count;                        // 0: none
  int route_rows;                   // 0: replicate; else rows per routed block (multiple of 256)
  int first_block;                  // route: the tile walk starts at this block (spreads the ranks' targets)
  long long ld;                     // elements between rows in every destination
  uint16_t* base[kMaxPeerCopies];   // replicate: element (0, 0) of D in destination i; route: row 0 of block i
};
// Validates and fills `out`; `tma_store` is the plan's store path (peer copies need it).
int set_peer_copies(PeerCopies* out, bool tma_store, int count, void* const* dst, long long ld, int N);
int set_row_route(PeerCopies* out, bool tma_store, int blocks, void* const* dst, int rows_per_block, long long ld,
                  int first_block, int M, int N);

// --------------------------------------------------------------------------- bf16 launch
struct Bf16Launch {
  CUtensorMap tmap_a, tmap_b, tmap_d;
  int M, N, K;
  int tile_n;        // width of one N sub-block: 64, 128 or 256
  int sub_blocks;    // N sub-blocks per tile: 1, or 2 (256 x 512 tiles, tile_n = 256 only)
  bool tma_store;    // false: D rows are not 16-byte aligned, use plain stores
  bool swiglu;       // gated epilogue: D is [M, N/2] = silu(acc[:, 1::2]) * acc[:, 0::2] (tma_store only)
  int group_m;       // raster group height (0 = default)
  int max_clusters;  // 0 = as many as fit
  void* d;
  int ldd;
  int* status;       // device status word, may be null
  long long* prof;   // device buffer of 8 counters per CTA (role timers), or null
  bool dynamic;      // tiles from the hardware work queue (cluster launch control) instead of a static walk
  bool operands_static;  // loads need not wait for the previous kernel on the stream
  bool output_independent;  // with operands_static: stores need not wait either
  PeerCopies peers;
  const int* mtile_group;  // grouped GEMM (device array, one group id per 256-row tile of A), or null
  // Grouped GEMM over groups of any row count (device arrays, one entry per row tile, or null):
  // first row of the tile and the row where its group ends.  tiles_m then comes from tile_rows.
  const int* tile_row0;
  const int* tile_row_end;
  int tile_rows;
  int l2_a, l2_b;    // L2 eviction hints of the A / BT loads: 0 none, 1 evict-last, 2 evict-first
  // Stream-K walk (gemm_bf16_streamk.cu): workspace for partial sums and flags (device, owned by
  // the plan), the number of clusters they have slots for, and this launch's number.  Null: whole tiles.
  float* streamk_partial;
  unsigned* streamk_flags;
  int streamk_clusters;
  unsigned streamk_epoch;
};
void bf16_pick_tile(int M, int N, int K, int clusters, int* tile_n, int* sub_blocks);
// Number of 2-CTA clusters that can run at once on the current device (SM count / 2), 0 if unknown.
int device_cluster_slots();
int bf16_launch(const Bf16Launch& L, cudaStream_t stream);
// The same GEMM with the tiles' K loops cut where the clusters' shares end (256 x 512 tiles, aligned
// plain store): whether it pays for a shape, what it needs, launch.
// The cut of the last wave: `full_waves` waves of whole tiles, then `rem_tiles` tiles whose K
// blocks [0, cut) go to one cluster each and [cut, end) to the spare clusters, `tails_per_cluster`
// tiles each (parts == 0), or which are cut into parts + 1 equal slices (parts > 0).
struct StreamKWalk {
  int full_waves, rem_tiles, cut, tails_per_cluster, parts;
};
double bf16_streamk_plan(long long tiles, int kb, int clusters, StreamKWalk* w);
bool bf16_streamk_pays(int M, int N, int K, int clusters);
size_t bf16_streamk_workspace_bytes(int clusters);
size_t bf16_streamk_flag_bytes(int clusters);
int bf16_streamk_launch(const Bf16Launch& L, cudaStream_t stream);

// --------------------------------------------------------------------------- nvfp4 launch
struct Fp4Launch {
  CUtensorMap tmap_a, tmap_b0, tmap_b1, tmap_sfa, tmap_sfb, tmap_d;
  int M, N, K;
  int w0, w1;        // widths of the tile's N sub-blocks (w1 = 0: one sub-block)
  bool tma_store;
  bool swiglu;       // gated epilogue (256-wide tiles only), as in Bf16Launch
  int group_m;
  int max_clusters;
  void* d;
  int ldd;
  int* status;
  long long* prof;
  int prefetch;      // L2 prefetch distance in K blocks (0 = off)
  bool dynamic;      // tiles from the hardware work queue instead of a static walk
  bool operands_static;  // loads need not wait for the previous kernel on the stream
  bool output_independent;  // with operands_static: stores need not wait either
  PeerCopies peers;
  const int* mtile_group;  // grouped GEMM (device array, one group id per 256-row tile of A), or null
  const int* tile_row0;    // as in Bf16Launch; group sizes multiples of 128 (scale bands)
  const int* tile_row_end;
  int tile_rows;
  bool block16;      // NVFP4 proper: UE4M3 scales per 16 K (256-wide tiles only)
  float alpha;       // factor on every accumulator (block16 only; 1 otherwise)
  bool uniform_tiles;  // true: full-width tiles only (no narrower tiles at the end of the tile list)
  int l2_a, l2_b;    // L2 eviction hints of the A / B loads: 0 none, 1 evict-last, 2 evict-first
};
void fp4_pick_tile(int M, int N, int K, int clusters, int* w0, int* w1);
void fp4_split_phases(int M, int N, int K, int w0, int w1, int clusters, int* wide_tiles_n, int* narrow_tiles_n);
int fp4_launch(const Fp4Launch& L, cudaStream_t stream);
// The A-resident schedule for short K (gemm_nvfp4_arun.cu; L.w0 == 192): whether a shape has it,
// how a tile row is cut into runs for `clusters` clusters (returns the estimated cycles), launch.
bool fp4_arun_supports(int M, int N, int K);
double fp4_arun_split(int M, int N, int K, int clusters, int* chunks, int* run_len);
int fp4_arun_launch(const Fp4Launch& L, cudaStream_t stream);

// --------------------------------------------------------------------------- nvfp4 decode launch
struct Fp4DecodeLaunch {
  CUtensorMap tmap_w, tmap_x, tmap_sfw, tmap_sfx;
  CUtensorMap tmap_d;   // D as [M, N] bf16, boxes of fp4_decode_box_rows(M) x 128, no swizzle (d_tma only)
  CUtensorMap tmap_d_rows;   // D as [M, N] bf16, boxes of 32 x 64, 128-byte swizzle (wide form, d_tma only)
  int M, N, K;       // M <= 128 activation rows, N weight rows
  void* d;
  int ldd;
  bool d_tma;        // false: D is not 16-byte aligned, every thread stores its own elements
  float* scratch;    // 2 * scratch_ctas slots of fp4_decode_slot_bytes(M); need no clearing
  int scratch_ctas;  // CTAs the scratch has slots for (caps the grid)
  int* counters;     // int  [ceil(N/128)], zero between calls
  int* status;
  int max_ctas;      // 0 = one per SM
  int max_stages;    // 0 = as many as fit
  bool no_overlap;   // true: plain stream order, no programmatic dependent launch
  bool activations_dynamic;  // X and its scales are written by the previous kernel on the stream
  bool dual;         // two weight tiles per activation box (whole tile pairs; ignored with max_ctas > 0)
  const void* act_src;  // BF16 activations [M, K] behind X (plans created from BF16 activations), or null
  long long act_ld;     // elements between their rows
  // How such a plan quantises: 0 = once per launch, shared by the CTAs of the decode kernel
  // (needs act_codes / act_sf / act_counter); 1 = inside every CTA for up to 16 rows, else a
  // kernel chained in front; 2 = always the kernel chained in front.
  int act_mode;
  void* act_codes;      // [M, K/2] codes and packed scales the kernel's tensor maps of X read
  void* act_sf;
  unsigned long long* act_counter;   // device, zero at plan creation
  bool narrow;       // true: never the wide form (activations as the instruction's rows) of the dual kernel
  bool block16;      // E4M3 scales per 16 K (dual form only); tmap_sfw / tmap_sfx boxes are 256 words
  float alpha;       // factor on every accumulator (block16 only)
  bool swiglu;       // gated epilogue: D is [M, N/2] = silu(acc[:, 1::2]) * acc[:, 0::2]; set before binding D
};
int fp4_decode_stage_bytes(int m_pad);
bool fp4_decode_prefers_dual(int M);   // default choice of Fp4DecodeLaunch::dual for M activation rows
bool fp4_decode_fuses_activations(const Fp4DecodeLaunch& L);   // the launch quantises L.act_src itself, per CTA
bool fp4_decode_spreads_activations(const Fp4DecodeLaunch& L); // ... itself, once per launch across the grid
size_t fp4_decode_slot_bytes(int M);                       // one fp32 partial tile
size_t fp4_decode_scratch_bytes(int M, int N, int ctas);   // slots for `ctas` CTAs + tile counters
int fp4_decode_box_rows(int M);
int fp4_decode_bind_output(Fp4DecodeLaunch* L, void* d, int M, int N, long long ldd, bool allow_tma);
// BF16 [rows, K] -> E2M1 codes + UE8M0 scales (packed and/or row-major).  `chained`: launched so
// that the next kernel on the stream may start early (see fills.cu).
int quantize_bf16_launch(const void* src, int64_t ld_src, void* data, int64_t ld_bytes, void* sf_packed,
                         void* sf_rowmajor, int64_t rows, int64_t K, bool chained, cudaStream_t st);
int fp4_decode_launch(const Fp4DecodeLaunch& L, cudaStream_t stream);

}  // namespace smb
