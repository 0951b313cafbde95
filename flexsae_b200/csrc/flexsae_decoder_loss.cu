// Fused TopK / Hierarchical-TopK decoder loss for B200 (sm_100a): forward, backward and the
// C ABI around them.
//
// Work decomposition.  Everything in both losses is independent along the model width D except
// two reductions (the loss sum and the dvals dot products), so D is cut into column PIECES of
// PW = G * VEC columns (VEC = elements per 16-byte load, G = 8/16/32 lanes that share one batch
// row) and the grid is ordered piece-major: all batch rows for piece 0, then piece 1, ...
// While one piece is being processed, the only decoder bytes touched are that piece's columns
// of all F rows (F*PW*sizeof(T)), and the only gradient bytes touched are an fp32 slab
// [F, PW].  G is chosen so that both stay resident in the 126 MB L2: the K gathers of a batch
// row then hit L2 (each decoder row is used by many batch rows), and the dweight scatter-add is
// resolved by the L2 atomic units without read-modify-write traffic to HBM.  After a piece is
// done the slab is converted to the decoder's storage type, written to dweight and cleared.
//
// One lane group walks the K active rows of its batch row in order (forward) or in reverse
// (backward) with the running reconstruction in registers, so the [B, K, D] tensor of prefix
// reconstructions never exists.  This mirrors what hierarchical_sae_forward_kernel /
// hierarchical_sae_backward_kernel compute (torch-ext/flex_sae/hierarchical_kernels.py:12-187)
// and, with the prefix removed, embedding_bag_forward_kernel and the TopK gradient
// (torch-ext/flex_sae/topk_kernels.py:15-41,97-137).
#include <stdarg.h>

#include <mutex>
#include <stdio.h>
#include <string.h>

#include "flexsae_common.cuh"
#include "flexsae_deterministic.cuh"
#include "flexsae_kernel_args.cuh"

namespace flexsae {

// ---- tuning state ------------------------------------------------------------------------------
struct Options {
  int lanes_fwd = 0;      // 0 = auto
  int lanes_bwd = 0;      // 0 = auto
  int lanes_sharded = 0;  // batch-sharded backward; 0 = lanes_bwd if that is set, else auto with 1.5 x the L2 budget
  int l2_budget_mb = 80;  // one piece of decoder columns (+ its fp32 slabs) must fit in this many MiB
  int segments = 0;       // K-segments per batch row in the backward; 0 = auto
  int pipeline = 1;       // 1: all column pieces of the atomic backward in one launch; 0: one launch per piece
  int convert_offset_pct = 60;  // where, inside a piece's unit blocks, the previous piece's converters sit
  int exchange_blocks = 148;    // sharded backward: blocks per slot for the cross-GPU reduce / broadcast / copy
  int exchange_offset_pct = 0;  // ... and where inside a piece's unit blocks they sit (capped at convert_offset_pct)
  int scatter_rotate = -1;      // sharded backward: ranks start their scatter sweeps at different row blocks (-1: from 4 ranks up)
  int sharded_convert_blocks = 0;       // sharded backward: converting blocks per piece (0 = as on one GPU)
  int sharded_convert_offset_pct = 45;  // sharded backward: their place in the piece (-1 = convert_offset_pct); their work
                                        // includes the NVLink stores, so they start earlier: 1.3 % per step at 2 and 4 GPUs
  int flag_fan_out = -1;        // sharded backward: a finished slot is announced by one thread per rank (-1: from 4 ranks up)
  int direct_f32 = 1;           // fp32 decoder: reduce straight into dweight instead of slab + copy
  int ticket_order = 0;         // single-launch kernels: blocks take their roles in the order they start (atomic ticket)
  int slabs = 2;                // fp32 accumulation slabs in rotation (2..4)
  int convert_lag = 1;          // slot p converts the slab of piece p - convert_lag (1 .. slabs-1)
  int wait_limit_ms = 5000;     // how long one in-kernel wait (for other blocks, for other GPUs) may last
};
static Options g_opt;

static thread_local char t_err[512] = "";
static thread_local int t_launches = 0;

static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err, sizeof(t_err), fmt, ap);
  va_end(ap);
  return code;
}

static size_t dtype_size(int dt) { return dt == FLEXSAE_F32 ? 4 : 2; }
static bool dtype_ok(int dt) { return dt == FLEXSAE_F32 || dt == FLEXSAE_BF16 || dt == FLEXSAE_F16; }
static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace flexsae

#include "flexsae_forward.cuh"
#include "flexsae_backward.cuh"
#include "flexsae_sharded.cuh"
#include "flexsae_small_allreduce.cuh"
#include "flexsae_topk_select.cuh"
#include "flexsae_index_skew.cuh"

namespace flexsae {

// ---- host side -------------------------------------------------------------------------------------
struct Shape {
  int64_t B, K, F, D;
};

static int check_shape(int kind, const Shape& s, int wdt) {
  if (kind != FLEXSAE_TOPK && kind != FLEXSAE_HIER) return fail(FLEXSAE_EINVAL, "unknown loss kind %d", kind);
  if (!dtype_ok(wdt)) return fail(FLEXSAE_EINVAL, "unknown weight dtype code %d", wdt);
  if (s.B < 1 || s.K < 1 || s.F < 1 || s.D < 1)
    return fail(FLEXSAE_EINVAL, "B, K, F, D must be positive (got %lld %lld %lld %lld)", (long long)s.B, (long long)s.K,
                (long long)s.F, (long long)s.D);
  const int vec = 16 / (int)dtype_size(wdt);
  if (s.D % vec != 0)
    return fail(FLEXSAE_EUNSUPPORTED, "D=%lld must be a multiple of %d (16-byte row pieces)", (long long)s.D, vec);
  if (s.F > (1ll << 30) || s.D > (1ll << 20) || s.B > (1ll << 27) || s.B * s.K > (1ll << 31) - 1)
    return fail(FLEXSAE_EUNSUPPORTED, "shape too large for 32-bit row/position arithmetic");
  // decoder rows are addressed in 16-byte units held in 32 bits: the table must stay below 2^36 bytes (64 GiB)
  if ((double)s.F * (double)s.D * (double)dtype_size(wdt) >= 68719476736.0)
    return fail(FLEXSAE_EUNSUPPORTED, "decoder of %lld x %lld elements is 64 GiB or more: beyond the 32-bit row-piece offsets",
                (long long)s.F, (long long)s.D);
  // 8 (+4 in deterministic mode) bytes per (unit, step) are staged in shared memory next to the
  // 32 KiB row-piece ring: 16 units * K * 12 bytes must fit
  if (s.K > 960) return fail(FLEXSAE_EUNSUPPORTED, "K=%lld above the supported maximum of 960", (long long)s.K);
  return 0;
}

// lanes per batch row: the widest group whose per-piece working set -- the piece's decoder columns
// plus, in the backward, all fp32 slabs in rotation -- fits the L2 budget
static int choose_lanes(int64_t F, int wdt, bool with_slab, int forced, double budget_scale = 1.0) {
  if (forced == 8 || forced == 16 || forced == 32) return forced;
  const int vec = 16 / (int)dtype_size(wdt);
  const double budget = (double)g_opt.l2_budget_mb * 1048576.0 * budget_scale;
  // an fp32 decoder accumulates straight into its dweight columns: one fp32 table instead of the slabs
  const int tables = !with_slab ? 0 : ((wdt == FLEXSAE_F32 && g_opt.direct_f32 && g_opt.pipeline) ? 1 : g_opt.slabs);
  auto bytes = [&](int G) { return (double)F * G * vec * (dtype_size(wdt) + 4.0 * tables); };
  for (int G = 32; G >= 8; G >>= 1)
    if (bytes(G) <= budget) return G;
  // nothing fits: the narrowest pieces while they are within reach of the L2, else stream from HBM
  // with the widest (most coalesced) row pieces
  return bytes(8) <= 2.0 * budget ? 8 : 32;
}

// Share of the L2 budget the single-GPU atomic backward may use.  The dense cost of a column piece
// (clearing and converting its fp32 slab, and the slab lines that spill to HBM once two slabs exceed
// about half the L2) does not depend on the batch; the cost per contribution falls with wider
// pieces.  Measured at F=65536, D=2304, bf16, uniform indices, 8 / 16 lanes in ms per fwd+bwd:
// B*K/F = 2: 0.75 / 0.87; 4: 1.02 / 1.15; 8: 1.54 / 1.56; 16: 2.70 / 2.47; 32: 4.78 / 4.34.  So up
// to 8 contributions per decoder row the slabs have to fit 4/5 of the budget (64 of 80 MiB).
static double bwd_budget_scale(const Shape& s) { return (double)s.B * (double)s.K > 8.0 * (double)s.F ? 1.0 : 0.8; }

static int round_up(int x, int m) { return (x + m - 1) / m * m; }

// segment length for a requested number of K-segments, and the count that length gives
static void segment_layout(int K, int want, int* KS, int* NS) {
  if (want < 1) want = 1;
  int ks = round_up((K + want - 1) / want, kUnroll);
  *KS = ks;
  *NS = (K + ks - 1) / ks;
}

// K-segments so that one column piece of the backward offers about a full machine of warps
static int choose_segments(const Shape& s, int wdt) {
  int want = g_opt.segments;
  if (want <= 0) {
    const int G = choose_lanes(s.F, wdt, true, g_opt.lanes_bwd, bwd_budget_scale(s));
    const double warps = (double)s.B * G / 32.0;
    const double target = 148.0 * 32.0;
    want = (int)((target + warps - 1) / warps);
    if (want > 8) want = 8;
  }
  int KS, NS;
  segment_layout((int)s.K, want, &KS, &NS);
  if (g_opt.segments <= 0 && (long long)NS * KS != s.K) {
    // prefer the next larger count whose segments tile K exactly: padding steps are wasted work
    for (int w = want + 1; w <= 8; w++) {
      int ks, ns;
      segment_layout((int)s.K, w, &ks, &ns);
      if ((long long)ns * ks == s.K) return ns;
    }
  }
  return NS;
}

static size_t state_floats(int kind, const Shape& s, int NS) {
  return (size_t)s.B * s.D * ((kind == FLEXSAE_HIER && NS > 1) ? 2 * (size_t)NS : 1);
}

static int check_segments(int kind, const Shape& s, int segments, int* KS, int* NS) {
  if (segments < 1) return fail(FLEXSAE_EINVAL, "segments must be >= 1 (got %d)", segments);
  segment_layout((int)s.K, segments, KS, NS);
  if (*NS != segments)
    return fail(FLEXSAE_EINVAL, "segments=%d is not a layout of K=%lld (use flexsae_choose_segments; nearest is %d)",
                segments, (long long)s.K, *NS);
  return 0;
}

constexpr int kMaxRowBlocks = 128;  // partial rows of the dbias column sums
constexpr int kConvertBlocks = FLEXSAE_CONVERT_BLOCKS;  // CTAs per piece that convert the previous piece's slab

// Counters of the single-launch kernels: four arrays of one int per slot (a launch has at most
// pieces + kMaxSlabs + 1 slots) and the ticket.
static size_t counter_stride(int pieces) { return (size_t)pieces + kMaxSlabs + 2; }
static size_t counter_ints(int pieces) { return 4 * counter_stride(pieces) + 2; }

struct BwdPlan {
  int G, PW, pieces, row_blocks, rows_per_block;
  size_t slab_bytes, stage_bytes, part_bytes, off_slab, off_dv, off_db, off_s0, off_ctr, off_index, off_stage, off_part, total;
};

// `sharded`: the plan of flexsae_loss_bwd_sharded.  Its slots carry a cross-GPU hand-shake each, so
// wider (fewer) pieces pay even more than on one GPU: measured on two GPUs at the headline shape,
// 16 lanes 1.69 ms per step against 1.78 with 8.  Hence half as much again of the L2 budget, and
// its own override.  `wide`: 32 lanes whatever fits (FLEXSAE_DW_ATOMIC_WIDE, for skewed indices: with
// Zipf indices every column piece repeats the serialised reductions into the hot decoder rows, 5.8 ms
// with 8 lanes against 3.7 with 16 and 3.0 with 32 at config 4).
static BwdPlan plan_bwd(const Shape& s, int wdt, int dw_mode, bool sharded = false, bool wide = false) {
  BwdPlan p;
  p.stage_bytes = p.part_bytes = 0;
  const int vec = 16 / (int)dtype_size(wdt);
  // deterministic mode keeps no fp32 slab in L2 (its contributions stream through a staging buffer),
  // so only the decoder columns count, and wider pieces mean fewer launches and longer staged rows
  p.G = sharded ? choose_lanes(s.F, wdt, true, g_opt.lanes_sharded ? g_opt.lanes_sharded : g_opt.lanes_bwd, 1.5)
                : choose_lanes(s.F, wdt, dw_mode == FLEXSAE_DW_ATOMIC, g_opt.lanes_bwd ? g_opt.lanes_bwd : (wide ? 32 : 0),
                               dw_mode == FLEXSAE_DW_ATOMIC ? bwd_budget_scale(s) : 1.0);
  p.PW = p.G * vec;
  p.pieces = (int)((s.D + p.PW - 1) / p.PW);
  p.rows_per_block = (int)((s.B + kMaxRowBlocks - 1) / kMaxRowBlocks);
  if (p.rows_per_block < 32) p.rows_per_block = 32;
  p.row_blocks = (int)((s.B + p.rows_per_block - 1) / p.rows_per_block);
  size_t off = 0;
  p.off_slab = off;  // the slabs in rotation: one accumulating, the others being converted or waiting for it
  p.slab_bytes = dw_mode == FLEXSAE_DW_ATOMIC ? align_up((size_t)s.F * p.PW * 4, 256) : 0;
  off += (size_t)g_opt.slabs * p.slab_bytes;
  p.off_index = p.off_stage = p.off_part = off;
  if (dw_mode == FLEXSAE_DW_DETERMINISTIC) {
    const int64_t n = s.B * s.K;
    off += det_index_bytes(n, s.F);
    p.off_stage = off;  // the staged contribution rows of one column piece
    p.stage_bytes = align_up((size_t)n * p.PW * 4, 256);
    off += p.stage_bytes;
    p.off_part = off;
    p.part_bytes = align_up(det_part_rows(n, s.F) * p.PW * 4, 256);
    off += p.part_bytes;
  }
  p.off_dv = off;
  off = align_up(off + (size_t)p.pieces * s.B * s.K * 4, 256);
  p.off_db = off;
  off = align_up(off + (size_t)p.row_blocks * s.D * 4, 256);
  p.off_s0 = off;  // summed prefix residuals of every row (Hierarchical; TopK does not use it)
  off = align_up(off + (size_t)s.B * s.D * 4, 256);
  p.off_ctr = off;  // per-piece completion counters of the single-launch pipeline
  off = align_up(off + counter_ints(p.pieces) * 4, 256);
  p.total = off;
  return p;
}

struct FwdPlan {
  int G, PW, pieces;
  size_t total;
};

static FwdPlan plan_fwd(const Shape& s, int wdt) {
  FwdPlan p;
  const int vec = 16 / (int)dtype_size(wdt);
  p.G = choose_lanes(s.F, wdt, false, g_opt.lanes_fwd);
  p.PW = p.G * vec;
  p.pieces = (int)((s.D + p.PW - 1) / p.PW);
  p.total = align_up((size_t)p.pieces * s.B * 4, 256);
  return p;
}

constexpr size_t kRingBytes = (size_t)kRingSlots * kThreads * sizeof(uint4);  // 2 KiB per slot and CTA

// Dynamic plus static shared memory above 48 KiB needs the opt-in attribute; the kernels declare a few
// bytes of static shared memory themselves, so the opt-in is asked for a little below the line.
template <typename K>
static cudaError_t allow_smem(K kern, size_t smem) {
  if (smem <= 40 * 1024) return cudaSuccess;
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
}

template <typename T, int G, bool HIER, bool SEG>
static cudaError_t launch_fwd_seg(const FwdArgs& a, int pieces, cudaStream_t st) {
  constexpr int RPC = groups_per_cta(G);
  const size_t smem = (size_t)RPC * ((a.K + kUnroll - 1) / kUnroll * kUnroll) * sizeof(int2);
  auto kern = decoder_loss_fwd_kernel<T, G, HIER, SEG>;
  if (cudaError_t e = allow_smem(kern, smem)) return e;
  dim3 grid((a.B + RPC - 1) / RPC, pieces);
  kern<<<grid, kThreads, smem, st>>>(a);
  t_launches++;
  return cudaGetLastError();
}

template <typename T, int G, bool HIER>
static cudaError_t launch_fwd(const FwdArgs& a, int pieces, cudaStream_t st) {
  if (HIER && a.NS > 1) return launch_fwd_seg<T, G, HIER, true>(a, pieces, st);
  return launch_fwd_seg<T, G, HIER, false>(a, pieces, st);
}

template <typename T, int G, bool HIER>
static cudaError_t launch_bwd_det(BwdArgs a, cudaStream_t st) {
  constexpr int UPC = groups_per_cta(G);
  const size_t smem = kRingBytes + (size_t)UPC * a.KS * (sizeof(int2) + sizeof(int));
  auto kern = decoder_loss_bwd_kernel<T, G, HIER, true>;
  if (cudaError_t e = allow_smem(kern, smem)) return e;
  const long long units = (long long)a.B * a.NS;
  a.unit_blocks = (int)((units + UPC - 1) / UPC);
  a.conv_blocks = 0;
  a.conv_stride = 1;
  kern<<<a.unit_blocks, kThreads, smem, st>>>(a);
  t_launches++;
  return cudaGetLastError();
}

template <typename T, int G, bool HIER>
static cudaError_t launch_bwd(BwdArgs a, cudaStream_t st) {
  constexpr int UPC = groups_per_cta(G);
  const size_t smem = kRingBytes + (size_t)UPC * a.KS * sizeof(int2);
  auto kern = decoder_loss_bwd_kernel<T, G, HIER, false>;
  if (cudaError_t e = allow_smem(kern, smem)) return e;
  const long long units = (long long)a.B * a.NS;
  a.unit_blocks = a.piece >= 0 ? (int)((units + UPC - 1) / UPC) : 0;
  int conv_blocks = 0;
  if (a.conv_piece >= 0) {
    const long long items = (long long)a.F * G;
    conv_blocks = (int)((items + kThreads * 4 - 1) / (kThreads * 4));
    const int cap = a.piece >= 0 ? kConvertBlocks : kConvertBlocks * 4;
    if (conv_blocks > cap) conv_blocks = cap;
  }
  a.conv_blocks = conv_blocks;
  a.conv_stride = conv_blocks > 0 ? (a.unit_blocks + conv_blocks) / conv_blocks : 1;
  kern<<<a.unit_blocks + conv_blocks, kThreads, smem, st>>>(a);
  t_launches++;
  return cudaGetLastError();
}

static void fill_pipe_args(PipeArgs& pa, const BwdArgs& b, float* const* slabs, int* counters, int pieces, int UPC) {
  pa.b = b;
  for (int i = 0; i < kMaxSlabs; i++) pa.slabs[i] = i < g_opt.slabs ? slabs[i] : nullptr;
  pa.nslabs = g_opt.slabs;
  pa.conv_lag = g_opt.convert_lag;
  pa.walk_done = counters;
  pa.conv_done = counters + counter_stride(pieces);
  pa.ticket = g_opt.ticket_order ? counters + 4 * counter_stride(pieces) : nullptr;
  pa.pieces = pieces;
  pa.wait_ns = (long long)g_opt.wait_limit_ms * 1000000ll;
  const long long units = (long long)b.B * b.NS;
  pa.unit_blocks = (int)((units + UPC - 1) / UPC);
}

template <typename T, int G, bool HIER>
static cudaError_t launch_bwd_pipelined(const BwdArgs& b, float* const* slabs, int* counters, int pieces, bool direct,
                                        cudaStream_t st) {
  constexpr int UPC = groups_per_cta(G);
  const size_t smem = kRingBytes + (size_t)UPC * b.KS * sizeof(int2);
  auto kern = decoder_loss_bwd_pipelined_kernel<T, G, HIER>;
  if (cudaError_t e = allow_smem(kern, smem)) return e;
  PipeArgs pa;
  fill_pipe_args(pa, b, slabs, counters, pieces, UPC);
  const long long items = (long long)b.F * G;
  int conv = (int)((items + kThreads * 4 - 1) / (kThreads * 4));
  if (conv > kConvertBlocks) conv = kConvertBlocks;
  if (direct) conv = 0;
  pa.conv_blocks = conv;
  pa.conv_offset = (int)((long long)pa.unit_blocks * g_opt.convert_offset_pct / 100);
  const long long blocks = (long long)pieces * (pa.unit_blocks + conv) + (long long)pa.conv_lag * conv;
  if (blocks > 0x7fffffffll) return cudaErrorInvalidConfiguration;
  kern<<<(unsigned)blocks, kThreads, smem, st>>>(pa);
  t_launches++;
  return cudaGetLastError();
}

template <typename T, int G, bool HIER>
static cudaError_t launch_bwd_sharded(const BwdArgs& b, float* const* slabs, int* counters, int pieces, ShardArgs sa,
                                      cudaStream_t st) {
  constexpr int UPC = groups_per_cta(G);
  const size_t smem = kRingBytes + (size_t)UPC * b.KS * sizeof(int2);
  auto kern = decoder_loss_bwd_sharded_kernel<T, G, HIER>;
  if (cudaError_t e = allow_smem(kern, smem)) return e;
  PipeArgs& pa = sa.p;
  fill_pipe_args(pa, b, slabs, counters, pieces, UPC);           // conv_done: one counter per slot here
  sa.slot_done = counters + 2 * counter_stride(pieces);
  sa.scatter_done = counters + 3 * counter_stride(pieces);
  const long long items = (long long)b.F * G;
  int conv = (int)((items + kThreads * 4 - 1) / (kThreads * 4));
  const int conv_cap = g_opt.sharded_convert_blocks > 0 ? g_opt.sharded_convert_blocks : kConvertBlocks;
  if (conv > conv_cap) conv = conv_cap;
  pa.conv_blocks = conv;
  const int conv_pct = g_opt.sharded_convert_offset_pct >= 0 ? g_opt.sharded_convert_offset_pct : g_opt.convert_offset_pct;
  pa.conv_offset = (int)((long long)pa.unit_blocks * conv_pct / 100);
  sa.exch_blocks = g_opt.exchange_blocks;
  sa.exch_offset = (int)((long long)pa.unit_blocks * g_opt.exchange_offset_pct / 100);
  if (sa.exch_offset > pa.conv_offset) sa.exch_offset = pa.conv_offset;
  // measured: the rotated sweep and the parallel flag updates cost 3 % on two GPUs and gain 3 % on four
  sa.rotate = g_opt.scatter_rotate >= 0 ? g_opt.scatter_rotate : (sa.world >= 4);
  sa.fan_out = g_opt.flag_fan_out >= 0 ? g_opt.flag_fan_out : (sa.world >= 4);
  const long long blocks = (long long)pieces * (sa.exch_blocks + pa.unit_blocks + conv) +
                           (long long)(pa.conv_lag + 2) * (sa.exch_blocks + conv);
  if (blocks > 0x7fffffffll) return cudaErrorInvalidConfiguration;
  kern<<<(unsigned)blocks, kThreads, smem, st>>>(sa);
  t_launches++;
  return cudaGetLastError();
}

// dispatch over (element type, lanes, loss kind)
#define FLEXSAE_DISPATCH_G(T, G, kind, CALL) ((kind) == FLEXSAE_HIER ? CALL(T, G, true) : CALL(T, G, false))
#define FLEXSAE_DISPATCH_T(T, G, kind, CALL)                                                       \
  ((G) == 32 ? FLEXSAE_DISPATCH_G(T, 32, kind, CALL)                                               \
             : ((G) == 16 ? FLEXSAE_DISPATCH_G(T, 16, kind, CALL) : FLEXSAE_DISPATCH_G(T, 8, kind, CALL)))
#define FLEXSAE_DISPATCH(wdt, G, kind, CALL)                                                       \
  ((wdt) == FLEXSAE_F32 ? FLEXSAE_DISPATCH_T(float, G, kind, CALL)                                 \
                        : ((wdt) == FLEXSAE_BF16 ? FLEXSAE_DISPATCH_T(__nv_bfloat16, G, kind, CALL) \
                                                 : FLEXSAE_DISPATCH_T(__half, G, kind, CALL)))

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace flexsae

using namespace flexsae;

extern "C" {

int flexsae_version(void) { return 300; }

const char* flexsae_last_error(void) { return t_err; }

int flexsae_last_launch_count(void) { return t_launches; }

int flexsae_set_option(const char* name, int64_t value) {
  if (!name) return fail(FLEXSAE_EINVAL, "option name is null");
  const bool lanes_ok = value == 0 || value == 8 || value == 16 || value == 32;
  if (!strcmp(name, "lanes_fwd") && lanes_ok) { g_opt.lanes_fwd = (int)value; return 0; }
  if (!strcmp(name, "lanes_bwd") && lanes_ok) { g_opt.lanes_bwd = (int)value; return 0; }
  if (!strcmp(name, "lanes_sharded") && lanes_ok) { g_opt.lanes_sharded = (int)value; return 0; }
  if (!strcmp(name, "l2_budget_mb") && value >= 1 && value <= 4096) { g_opt.l2_budget_mb = (int)value; return 0; }
  if (!strcmp(name, "segments") && value >= 0 && value <= 256) { g_opt.segments = (int)value; return 0; }
  if (!strcmp(name, "pipeline") && (value == 0 || value == 1)) { g_opt.pipeline = (int)value; return 0; }
  if (!strcmp(name, "slabs") && value >= 2 && value <= kMaxSlabs) {
    g_opt.slabs = (int)value;
    if (g_opt.convert_lag > g_opt.slabs - 1) g_opt.convert_lag = g_opt.slabs - 1;
    return 0;
  }
  if (!strcmp(name, "convert_lag") && value >= 1 && value <= g_opt.slabs - 1) { g_opt.convert_lag = (int)value; return 0; }
  if (!strcmp(name, "ticket_order") && (value == 0 || value == 1)) { g_opt.ticket_order = (int)value; return 0; }
  if (!strcmp(name, "convert_offset_pct") && value >= 0 && value <= 100) { g_opt.convert_offset_pct = (int)value; return 0; }
  if (!strcmp(name, "direct_f32") && (value == 0 || value == 1)) { g_opt.direct_f32 = (int)value; return 0; }
  if (!strcmp(name, "exchange_blocks") && value >= 1 && value <= 4096) { g_opt.exchange_blocks = (int)value; return 0; }
  if (!strcmp(name, "exchange_offset_pct") && value >= 0 && value <= 100) { g_opt.exchange_offset_pct = (int)value; return 0; }
  if (!strcmp(name, "scatter_rotate") && value >= -1 && value <= 1) { g_opt.scatter_rotate = (int)value; return 0; }
  if (!strcmp(name, "flag_fan_out") && value >= -1 && value <= 1) { g_opt.flag_fan_out = (int)value; return 0; }
  if (!strcmp(name, "sharded_convert_blocks") && value >= 0 && value <= 8192) { g_opt.sharded_convert_blocks = (int)value; return 0; }
  if (!strcmp(name, "sharded_convert_offset_pct") && value >= -1 && value <= 100) { g_opt.sharded_convert_offset_pct = (int)value; return 0; }
  if (!strcmp(name, "wait_limit_ms") && value >= 1 && value <= 600000) { g_opt.wait_limit_ms = (int)value; return 0; }
  return fail(FLEXSAE_EINVAL, "unknown option or value: %s=%lld", name, (long long)value);
}

int64_t flexsae_get_option(const char* name) {
  if (!name) return -1;
  if (!strcmp(name, "lanes_fwd")) return g_opt.lanes_fwd;
  if (!strcmp(name, "lanes_bwd")) return g_opt.lanes_bwd;
  if (!strcmp(name, "lanes_sharded")) return g_opt.lanes_sharded;
  if (!strcmp(name, "l2_budget_mb")) return g_opt.l2_budget_mb;
  if (!strcmp(name, "segments")) return g_opt.segments;
  if (!strcmp(name, "pipeline")) return g_opt.pipeline;
  if (!strcmp(name, "slabs")) return g_opt.slabs;
  if (!strcmp(name, "convert_lag")) return g_opt.convert_lag;
  if (!strcmp(name, "ticket_order")) return g_opt.ticket_order;
  if (!strcmp(name, "convert_offset_pct")) return g_opt.convert_offset_pct;
  if (!strcmp(name, "direct_f32")) return g_opt.direct_f32;
  if (!strcmp(name, "exchange_blocks")) return g_opt.exchange_blocks;
  if (!strcmp(name, "exchange_offset_pct")) return g_opt.exchange_offset_pct;
  if (!strcmp(name, "scatter_rotate")) return g_opt.scatter_rotate;
  if (!strcmp(name, "flag_fan_out")) return g_opt.flag_fan_out;
  if (!strcmp(name, "sharded_convert_blocks")) return g_opt.sharded_convert_blocks;
  if (!strcmp(name, "sharded_convert_offset_pct")) return g_opt.sharded_convert_offset_pct;
  if (!strcmp(name, "wait_limit_ms")) return g_opt.wait_limit_ms;
  return -1;
}

int flexsae_choose_segments(int kind, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype) {
  Shape s{B, K, F, D};
  if (check_shape(kind, s, weight_dtype)) return 0;
  return choose_segments(s, weight_dtype);
}

size_t flexsae_state_bytes(int kind, int64_t B, int64_t K, int64_t D, int segments) {
  if ((kind != FLEXSAE_TOPK && kind != FLEXSAE_HIER) || B < 1 || K < 1 || D < 1 || segments < 1) return 0;
  Shape s{B, K, 1, D};
  return state_floats(kind, s, segments) * sizeof(float);
}

size_t flexsae_fwd_workspace_bytes(int kind, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype) {
  Shape s{B, K, F, D};
  if (check_shape(kind, s, weight_dtype)) return 0;
  return plan_fwd(s, weight_dtype).total;
}

size_t flexsae_bwd_workspace_bytes(int kind, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype, int dw_mode) {
  Shape s{B, K, F, D};
  if (check_shape(kind, s, weight_dtype)) return 0;
  if (dw_mode == FLEXSAE_DW_ATOMIC_SHARDED) return plan_bwd(s, weight_dtype, FLEXSAE_DW_ATOMIC, true).total;
  if (dw_mode == FLEXSAE_DW_ATOMIC_WIDE) return plan_bwd(s, weight_dtype, FLEXSAE_DW_ATOMIC, false, true).total;
  if (dw_mode != FLEXSAE_DW_ATOMIC && dw_mode != FLEXSAE_DW_DETERMINISTIC) {
    fail(FLEXSAE_EINVAL, "unknown dweight mode %d", dw_mode);
    return 0;
  }
  return plan_bwd(s, weight_dtype, dw_mode).total;
}

int flexsae_loss_fwd(int kind, const int64_t* indices, const void* weight, const void* vals, const void* bias,
                     const void* target, float* loss_out, float* state_out, int segments, void* workspace,
                     size_t workspace_bytes, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype,
                     int vals_dtype, int bias_dtype, int target_dtype, double inv_norm, int32_t* status, void* stream) {
  t_launches = 0;
  Shape s{B, K, F, D};
  if (int rc = check_shape(kind, s, weight_dtype)) return rc;
  if (!dtype_ok(vals_dtype) || !dtype_ok(bias_dtype) || !dtype_ok(target_dtype))
    return fail(FLEXSAE_EINVAL, "unknown dtype code (vals %d, bias %d, target %d)", vals_dtype, bias_dtype, target_dtype);
  int KS, NS;
  if (int rc = check_segments(kind, s, segments, &KS, &NS)) return rc;
  if (!indices || !weight || !vals || !bias || !target || !loss_out || !state_out || !workspace)
    return fail(FLEXSAE_EINVAL, "null pointer argument");
  if (!aligned16(weight) || !aligned16(bias) || !aligned16(target) || !aligned16(state_out) || !aligned16(workspace))
    return fail(FLEXSAE_EINVAL, "weight, bias, target, state and workspace must be 16-byte aligned");
  const FwdPlan p = plan_fwd(s, weight_dtype);
  if (workspace_bytes < p.total)
    return fail(FLEXSAE_EWORKSPACE, "forward workspace too small: %zu < %zu bytes", workspace_bytes, p.total);
  if (inv_norm <= 0.0) inv_norm = 1.0 / ((double)B * (double)D * (kind == FLEXSAE_HIER ? (double)K : 1.0));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

  FwdArgs a;
  a.indices = indices; a.weight = weight; a.vals = vals; a.bias = bias; a.target = target;
  a.loss_part = reinterpret_cast<float*>(workspace);
  a.state = state_out; a.status = status;
  a.B = (int)B; a.K = (int)K; a.F = (int)F; a.D = (int)D;
  a.vals_dtype = vals_dtype; a.bias_dtype = bias_dtype; a.target_dtype = target_dtype;
  a.KS = (kind == FLEXSAE_HIER) ? KS : round_up((int)K, kUnroll);
  a.NS = (kind == FLEXSAE_HIER) ? NS : 1;

#define CALL_FWD(T, G, H) launch_fwd<T, G, H>(a, p.pieces, st)
  cudaError_t e = FLEXSAE_DISPATCH(weight_dtype, p.G, kind, CALL_FWD);
#undef CALL_FWD
  if (e != cudaSuccess) return fail((int)e, "forward launch failed: %s", cudaGetErrorString(e));
  loss_finalize_kernel<<<1, 1024, 0, st>>>(a.loss_part, (size_t)p.pieces * B, inv_norm, loss_out);
  t_launches++;
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail((int)e, "loss finalize launch failed: %s", cudaGetErrorString(e));
  return 0;
}

}  // extern "C"

namespace flexsae {
struct PeerInfo {  // batch-sharded call: who the other GPUs are and where their exchange buffers live
  int world, rank, seq_base;
  void* const* x;
  void* const* y;
  void* const* flags;
  void* mc_x;
  void* mc_y;
  void* const* dweight;  // every rank's dweight (peer-mapped), or NULL
};

static int loss_bwd_impl(int kind, const int64_t* indices, const void* weight, const void* vals, const float* state,
                         int segments, const float* grad_out, void* dweight, void* dvals, void* dbias, void* workspace,
                         size_t workspace_bytes, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype,
                         int vals_dtype, int bias_dtype, double inv_norm, int dw_mode, int32_t* status, void* stream,
                         const PeerInfo* peers) {
  t_launches = 0;
  Shape s{B, K, F, D};
  if (int rc = check_shape(kind, s, weight_dtype)) return rc;
  if (!dtype_ok(vals_dtype) || !dtype_ok(bias_dtype))
    return fail(FLEXSAE_EINVAL, "unknown dtype code (vals %d, bias %d)", vals_dtype, bias_dtype);
  const bool wide = dw_mode == FLEXSAE_DW_ATOMIC_WIDE && !peers;
  if (wide) dw_mode = FLEXSAE_DW_ATOMIC;
  if (dw_mode != FLEXSAE_DW_ATOMIC && dw_mode != FLEXSAE_DW_DETERMINISTIC)
    return fail(FLEXSAE_EINVAL, "unknown dweight mode %d", dw_mode);
  int KS, NS;
  if (int rc = check_segments(kind, s, segments, &KS, &NS)) return rc;
  if (!indices || !weight || !vals || !state || !grad_out || !dweight || !dvals || !dbias || !workspace)
    return fail(FLEXSAE_EINVAL, "null pointer argument");
  if (!aligned16(weight) || !aligned16(state) || !aligned16(dweight) || !aligned16(workspace))
    return fail(FLEXSAE_EINVAL, "weight, state, dweight and workspace must be 16-byte aligned");
  const BwdPlan p = plan_bwd(s, weight_dtype, dw_mode, peers != nullptr, wide);
  if (workspace_bytes < p.total)
    return fail(FLEXSAE_EWORKSPACE, "backward workspace too small: %zu < %zu bytes", workspace_bytes, p.total);
  if (inv_norm <= 0.0) inv_norm = 1.0 / ((double)B * (double)D * (kind == FLEXSAE_HIER ? (double)K : 1.0));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  char* ws = reinterpret_cast<char*>(workspace);

  BwdArgs a;
  a.indices = indices; a.weight = weight; a.vals = vals; a.state = state; a.grad_out = grad_out;
  float* slabs[kMaxSlabs];
  for (int i = 0; i < kMaxSlabs; i++) slabs[i] = reinterpret_cast<float*>(ws + p.off_slab + (size_t)(i < g_opt.slabs ? i : 0) * p.slab_bytes);
  a.dweight = dweight;
  a.stage = nullptr;
  a.slot_of = nullptr;
  a.s0 = reinterpret_cast<float*>(ws + p.off_s0);
  a.dv_part = reinterpret_cast<float*>(ws + p.off_dv);
  a.status = status;
  a.B = (int)B; a.K = (int)K; a.F = (int)F; a.D = (int)D;
  a.vals_dtype = vals_dtype;
  a.scale = (float)(2.0 * inv_norm);
  a.KS = KS; a.NS = NS;
  a.slab_stride = p.PW;
  float* db_part = reinterpret_cast<float*>(ws + p.off_db);
  // An fp32 decoder needs no fp32 slab: dweight itself is the accumulation target (single GPU,
  // single-launch form).
  const bool direct = weight_dtype == FLEXSAE_F32 && dw_mode == FLEXSAE_DW_ATOMIC && !peers && g_opt.pipeline &&
                      g_opt.direct_f32;

  cudaError_t e = cudaSuccess;
  if (dw_mode == FLEXSAE_DW_DETERMINISTIC) {
    // Sort the (decoder row, position) pairs once; then per column piece: the same reverse walk,
    // but every contribution row is stored to its sorted slot, and the rows of each decoder row
    // are added in slot order straight into dweight.
    DetIndex ix;
    e = det_prepare(indices, B * K, F, ws + p.off_index, &ix, st, &t_launches);
    if (e != cudaSuccess) return fail((int)e, "sort launches failed: %s", cudaGetErrorString(e));
    a.slot_of = ix.slot_of;
    a.slab = a.conv_slab = nullptr;
    a.conv_piece = -1;
    a.stage = reinterpret_cast<float*>(ws + p.off_stage);
    float* part = reinterpret_cast<float*>(ws + p.off_part);
    for (int i = 0; i < p.pieces; i++) {
      a.piece = i;
#define CALL_DET(T, G, H) launch_bwd_det<T, G, H>(a, st)
      e = FLEXSAE_DISPATCH(weight_dtype, p.G, kind, CALL_DET);
#undef CALL_DET
      if (e != cudaSuccess) return fail((int)e, "backward launch failed: %s", cudaGetErrorString(e));
      e = det_reduce_piece(weight_dtype, p.G, a.stage, ix, (int)F, (int)D, i, part, dweight, st, &t_launches);
      if (e != cudaSuccess) return fail((int)e, "ordered sum launch failed: %s", cudaGetErrorString(e));
    }
  } else {
  // Both slabs are cleared once here; afterwards every conversion leaves its slab cleared.
  // Launch i accumulates piece i into slab i%2 and converts piece i-1 out of the other slab;
  // one more launch converts the last piece.
  if (direct) {
    e = cudaMemsetAsync(dweight, 0, (size_t)F * D * sizeof(float), st);
    a.slab_stride = (int)D;
  } else {
    e = cudaMemsetAsync(slabs[0], 0, (size_t)g_opt.slabs * p.slab_bytes, st);
  }
  if (e != cudaSuccess) return fail((int)e, "gradient clear failed: %s", cudaGetErrorString(e));
  if (peers) {
    int* counters = reinterpret_cast<int*>(ws + p.off_ctr);
    e = cudaMemsetAsync(counters, 0, counter_ints(p.pieces) * 4, st);
    if (e != cudaSuccess) return fail((int)e, "counter clear failed: %s", cudaGetErrorString(e));
    a.piece = a.conv_piece = -1;
    a.slab = a.conv_slab = nullptr;
    a.unit_blocks = a.conv_blocks = 0;
    a.conv_stride = 1;
    ShardArgs sa;
    sa.world = peers->world;
    sa.rank = peers->rank;
    sa.seq_base = peers->seq_base;
    sa.rows_per_rank = (int)((F + peers->world - 1) / peers->world);
    sa.mc_inbox = peers->mc_x;
    sa.mc_gathered = peers->mc_y;
    for (int r = 0; r < kMaxRanks; r++) {
      sa.inbox[r] = r < peers->world ? peers->x[r] : nullptr;
      sa.gathered[r] = r < peers->world ? peers->y[r] : nullptr;
      sa.flags_at[r] = r < peers->world ? reinterpret_cast<int*>(peers->flags[r]) : nullptr;
      sa.dweight_at[r] = (peers->dweight && r < peers->world) ? peers->dweight[r] : nullptr;
    }
#define CALL_SHARD(T, G, H) launch_bwd_sharded<T, G, H>(a, slabs, counters, p.pieces, sa, st)
    e = FLEXSAE_DISPATCH(weight_dtype, p.G, kind, CALL_SHARD);
#undef CALL_SHARD
    if (e != cudaSuccess) return fail((int)e, "sharded backward launch failed: %s", cudaGetErrorString(e));
  } else if (g_opt.pipeline) {
    int* counters = reinterpret_cast<int*>(ws + p.off_ctr);
    e = cudaMemsetAsync(counters, 0, counter_ints(p.pieces) * 4, st);
    if (e != cudaSuccess) return fail((int)e, "counter clear failed: %s", cudaGetErrorString(e));
    a.piece = a.conv_piece = -1;
    a.slab = a.conv_slab = nullptr;
    a.unit_blocks = a.conv_blocks = 0;
    a.conv_stride = 1;
#define CALL_PIPE(T, G, H) launch_bwd_pipelined<T, G, H>(a, slabs, counters, p.pieces, direct, st)
    e = FLEXSAE_DISPATCH(weight_dtype, p.G, kind, CALL_PIPE);
#undef CALL_PIPE
    if (e != cudaSuccess) return fail((int)e, "pipelined backward launch failed: %s", cudaGetErrorString(e));
  } else
  for (int i = 0; i <= p.pieces; i++) {
    a.piece = i < p.pieces ? i : -1;
    a.conv_piece = i - 1;
    a.slab = slabs[i & 1];
    a.conv_slab = slabs[(i & 1) ^ 1];
#define CALL_BWD(T, G, H) launch_bwd<T, G, H>(a, st)
    e = FLEXSAE_DISPATCH(weight_dtype, p.G, kind, CALL_BWD);
#undef CALL_BWD
    if (e != cudaSuccess) return fail((int)e, "backward launch failed: %s", cudaGetErrorString(e));
  }
  }
  // dbias = coef * column sums of the final residual (TopK) or of the summed prefix residuals the
  // first-segment walkers left in s0 (Hierarchical): partial sums over row blocks, fixed order.
  const float* colsrc = kind == FLEXSAE_HIER ? a.s0 : state;
  column_sums_kernel<<<dim3((unsigned)((D + 127) / 128), p.row_blocks), 128, 0, st>>>(colsrc, (int)B, (int)D,
                                                                                      p.rows_per_block, db_part);
  t_launches++;
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail((int)e, "column sums launch failed: %s", cudaGetErrorString(e));
  const size_t BK = (size_t)B * K;
  const int dv_blocks = (int)((BK + 255) / 256);
  const int db_blocks = (int)((D + 255) / 256);
  grads_finalize_kernel<<<dv_blocks + db_blocks, 256, 0, st>>>(a.dv_part, p.pieces, BK, dvals, vals_dtype, db_part,
                                                             p.row_blocks, (int)D, dbias, bias_dtype, dv_blocks,
                                                             grad_out, a.scale);
  t_launches++;
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail((int)e, "gradient finalize launch failed: %s", cudaGetErrorString(e));
  return 0;
}
}  // namespace flexsae

extern "C" {

int flexsae_loss_bwd(int kind, const int64_t* indices, const void* weight, const void* vals, const float* state,
                     int segments, const float* grad_out, void* dweight, void* dvals, void* dbias, void* workspace,
                     size_t workspace_bytes, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype,
                     int vals_dtype, int bias_dtype, double inv_norm, int dw_mode, int32_t* status, void* stream) {
  return loss_bwd_impl(kind, indices, weight, vals, state, segments, grad_out, dweight, dvals, dbias, workspace,
                       workspace_bytes, B, K, F, D, weight_dtype, vals_dtype, bias_dtype, inv_norm, dw_mode, status,
                       stream, nullptr);
}

int flexsae_shard_buffer_bytes(int64_t F, int64_t D, int weight_dtype, int world, size_t* x_bytes, size_t* y_bytes,
                               size_t* flag_bytes) {
  Shape s{1, 1, F, D};
  if (int rc = check_shape(FLEXSAE_HIER, s, weight_dtype)) return rc;
  if (world < 2 || world > kMaxRanks) return fail(FLEXSAE_EINVAL, "world size %d outside [2, %d]", world, kMaxRanks);
  if (!x_bytes || !y_bytes || !flag_bytes) return fail(FLEXSAE_EINVAL, "null pointer argument");
  const BwdPlan p = plan_bwd(s, weight_dtype, FLEXSAE_DW_ATOMIC, true);
  const size_t rows_per_rank = (size_t)((F + world - 1) / world);
  *x_bytes = align_up(2 * (size_t)world * rows_per_rank * p.PW * dtype_size(weight_dtype), 256);  // inbox
  *y_bytes = *x_bytes;                                                                           // gather buffer
  *flag_bytes = 256;
  return 0;
}

int flexsae_loss_bwd_sharded(int kind, const int64_t* indices, const void* weight, const void* vals,
                             const float* state, int segments, const float* grad_out, void* dweight, void* dvals,
                             void* dbias, void* workspace, size_t workspace_bytes, int64_t B, int64_t K, int64_t F,
                             int64_t D, int weight_dtype, int vals_dtype, int bias_dtype, double inv_norm,
                             int32_t* status, void* stream, int world, int rank, int seq_base, void* const* x_ptrs,
                             void* const* y_ptrs, void* const* flag_ptrs, void* multicast_x, void* multicast_y,
                             void* const* dweight_ptrs) {
  if (world < 2 || world > kMaxRanks) return fail(FLEXSAE_EINVAL, "world size %d outside [2, %d]", world, kMaxRanks);
  if (rank < 0 || rank >= world) return fail(FLEXSAE_EINVAL, "rank %d outside [0, %d)", rank, world);
  if (!x_ptrs || !y_ptrs || !flag_ptrs) return fail(FLEXSAE_EINVAL, "null pointer argument");
  for (int r = 0; r < world; r++)
    if (!x_ptrs[r] || !y_ptrs[r] || !flag_ptrs[r] || !aligned16(x_ptrs[r]) || !aligned16(y_ptrs[r]))
      return fail(FLEXSAE_EINVAL, "exchange buffer of rank %d is null or not 16-byte aligned", r);
  if (seq_base < 1) return fail(FLEXSAE_EINVAL, "seq_base must be >= 1");
  if ((multicast_x == nullptr) != (multicast_y == nullptr) || !aligned16(multicast_x) || !aligned16(multicast_y))
    return fail(FLEXSAE_EINVAL, "multicast addresses must both be given (16-byte aligned) or both be NULL");
  if (dweight_ptrs) {
    if (multicast_x) return fail(FLEXSAE_EINVAL, "dweight_ptrs cannot be combined with the multicast path");
    for (int r = 0; r < world; r++)
      if (!dweight_ptrs[r] || !aligned16(dweight_ptrs[r]))
        return fail(FLEXSAE_EINVAL, "dweight of rank %d is null or not 16-byte aligned", r);
    if (dweight_ptrs[rank] != dweight)
      return fail(FLEXSAE_EINVAL, "dweight_ptrs[rank] must be this rank's dweight");
  }
  PeerInfo peers{world, rank, seq_base, x_ptrs, y_ptrs, flag_ptrs, multicast_x, multicast_y, dweight_ptrs};
  return loss_bwd_impl(kind, indices, weight, vals, state, segments, grad_out, dweight, dvals, dbias, workspace,
                       workspace_bytes, B, K, F, D, weight_dtype, vals_dtype, bias_dtype, inv_norm, FLEXSAE_DW_ATOMIC,
                       status, stream, &peers);
}

}  // extern "C"

namespace flexsae {
template <typename T>
static cudaError_t launch_topk_select(const SelectArgs& a, int64_t B, cudaStream_t st) {
  // one maximum per 16-byte vector of the row in shared memory, if the row is short enough for that
  // to leave four CTAs per SM (F = 65536 in bf16: 16 KiB)
  const size_t per_vec = sizeof(T) == 4 ? 4 : 2;
  const size_t vmax_bytes = (size_t)(a.F / (16 / (int)sizeof(T))) * per_vec;
  if (vmax_bytes <= 32 * 1024) {
    auto kern = topk_select_kernel<T, true>;  // with its 17 KiB of static shared memory this can pass 48 KiB
    if (cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * 1024)) return e;
    kern<<<(unsigned)B, kSelThreads, vmax_bytes, st>>>(a);
  } else {
    topk_select_kernel<T, false><<<(unsigned)B, kSelThreads, 0, st>>>(a);
  }
  t_launches++;
  return cudaGetLastError();
}
}  // namespace flexsae

extern "C" {

int flexsae_topk_select(const void* acts, int acts_dtype, int64_t B, int64_t F, int64_t K, int relu, void* vals,
                        int vals_dtype, int64_t* indices, void* stream) {
  t_launches = 0;
  if (!dtype_ok(acts_dtype) || !dtype_ok(vals_dtype))
    return fail(FLEXSAE_EINVAL, "unknown dtype code (activations %d, vals %d)", acts_dtype, vals_dtype);
  if (B < 1 || F < 1 || K < 1) return fail(FLEXSAE_EINVAL, "B, F, K must be positive (got %lld %lld %lld)", (long long)B, (long long)F, (long long)K);
  if (!acts || !vals || !indices) return fail(FLEXSAE_EINVAL, "null pointer argument");
  if (!aligned16(acts)) return fail(FLEXSAE_EINVAL, "activations must be 16-byte aligned");
  const int vec = 16 / (int)dtype_size(acts_dtype);
  if (F % vec != 0) return fail(FLEXSAE_EUNSUPPORTED, "F=%lld must be a multiple of %d (16-byte loads)", (long long)F, vec);
  if (K > F) return fail(FLEXSAE_EINVAL, "K=%lld exceeds F=%lld", (long long)K, (long long)F);
  if (K > kSelMaxK) return fail(FLEXSAE_EUNSUPPORTED, "K=%lld above the supported maximum of %d", (long long)K, kSelMaxK);
  if (F > (1ll << 30) || B > 0x7fffffffll) return fail(FLEXSAE_EUNSUPPORTED, "shape too large for 32-bit index arithmetic");
  SelectArgs a;
  a.acts = acts;
  a.vals = vals;
  a.indices = indices;
  a.F = (int)F;
  a.K = (int)K;
  a.Kp = 1;
  while (a.Kp < a.K) a.Kp <<= 1;
  a.vals_dtype = vals_dtype;
  a.relu = relu != 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = acts_dtype == FLEXSAE_F32    ? launch_topk_select<float>(a, B, st)
                  : acts_dtype == FLEXSAE_BF16 ? launch_topk_select<__nv_bfloat16>(a, B, st)
                                               : launch_topk_select<__half>(a, B, st);
  if (e != cudaSuccess) return fail((int)e, "top-K selection launch failed: %s", cudaGetErrorString(e));
  return 0;
}

int flexsae_small_allreduce_bytes(int world, int64_t capacity, size_t* bytes) {
  if (world < 2 || world > kMaxRanks) return fail(FLEXSAE_EINVAL, "world size %d outside [2, %d]", world, kMaxRanks);
  if (capacity < 1 || capacity > (1 << 24) || !bytes) return fail(FLEXSAE_EINVAL, "capacity %lld outside [1, 2^24] or null pointer", (long long)capacity);
  *bytes = align_up(kSmallFlagBytes + 2 * (size_t)world * (size_t)capacity * sizeof(float), 256);
  return 0;
}

int flexsae_small_allreduce(const void* in, void* out, int64_t n, int dtype, int world, int rank, int seq,
                            void* const* buf_ptrs, int64_t capacity, int32_t* status, void* stream) {
  t_launches = 0;
  if (world < 2 || world > kMaxRanks) return fail(FLEXSAE_EINVAL, "world size %d outside [2, %d]", world, kMaxRanks);
  if (rank < 0 || rank >= world) return fail(FLEXSAE_EINVAL, "rank %d outside [0, %d)", rank, world);
  if (!in || !out || !buf_ptrs) return fail(FLEXSAE_EINVAL, "null pointer argument");
  if (!dtype_ok(dtype)) return fail(FLEXSAE_EINVAL, "unknown dtype code %d", dtype);
  if (capacity < 1 || capacity > (1 << 24)) return fail(FLEXSAE_EINVAL, "capacity %lld outside [1, 2^24]", (long long)capacity);
  if (n < 1 || n > capacity) return fail(FLEXSAE_EINVAL, "n = %lld outside [1, capacity = %lld]", (long long)n, (long long)capacity);
  if (seq < 1) return fail(FLEXSAE_EINVAL, "seq must be >= 1");
  SmallReduceArgs a;
  a.in = in;
  a.out = out;
  a.n = (int)n;
  a.dtype = dtype;
  a.world = world;
  a.rank = rank;
  a.seq = seq;
  a.capacity = capacity;
  a.wait_ns = (long long)g_opt.wait_limit_ms * 1000000ll;
  a.status = status;
  for (int r = 0; r < kMaxRanks; r++) {
    a.buf[r] = r < world ? buf_ptrs[r] : nullptr;
    if (r < world && (!a.buf[r] || !aligned16(a.buf[r])))
      return fail(FLEXSAE_EINVAL, "exchange buffer of rank %d is null or not 16-byte aligned", r);
  }
  small_allreduce_kernel<<<1, kSmallThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  t_launches++;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail((int)e, "small all-reduce launch failed: %s", cudaGetErrorString(e));
  return 0;
}

#ifdef FLEXSAE_TRACE
// Tuning builds only: copy the current device's slot timeline of the sharded backward to the host
// (and clear it).  Synchronises the device.
int flexsae_debug_trace_read(unsigned long long* out, size_t bytes, int clear) {
  if (!out || bytes != sizeof(unsigned long long) * 64 * kTrFields) return fail(FLEXSAE_EINVAL, "trace table is %zu bytes", sizeof(unsigned long long) * 64 * kTrFields);
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(out, g_trace, bytes);
  if (e == cudaSuccess && clear) {
    static unsigned long long zeros[64 * kTrFields];
    e = cudaMemcpyToSymbol(g_trace, zeros, bytes);
  }
  if (e != cudaSuccess) return fail((int)e, "trace read failed: %s", cudaGetErrorString(e));
  return 0;
}
#endif

size_t flexsae_sort_workspace_bytes(int64_t n, int64_t F) {
  if (n < 1 || F < 1 || n > (1ll << 31) - 1 || F > (1ll << 30)) return 0;
  return det_index_bytes(n, F);
}

int flexsae_sort_by_decoder_row(const int64_t* indices, int64_t n, int64_t F, void* workspace, size_t workspace_bytes,
                                int32_t* order, int32_t* slot_of, int32_t* seg_begin, int32_t* item_begin, void* stream) {
  t_launches = 0;
  if (n < 1 || F < 1 || n > (1ll << 31) - 1 || F > (1ll << 30))
    return fail(FLEXSAE_EINVAL, "n = %lld positions / F = %lld decoder rows outside the supported range", (long long)n, (long long)F);
  if (!indices || !workspace) return fail(FLEXSAE_EINVAL, "null pointer argument");
  if (!aligned16(workspace)) return fail(FLEXSAE_EINVAL, "workspace must be 16-byte aligned");
  const size_t need = det_index_bytes(n, F);
  if (workspace_bytes < need) return fail(FLEXSAE_EWORKSPACE, "sort workspace too small: %zu < %zu bytes", workspace_bytes, need);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  DetIndex ix;
  cudaError_t e = det_prepare(indices, n, F, reinterpret_cast<char*>(workspace), &ix, st, &t_launches);
  const size_t nb = (size_t)n * 4, fb = (size_t)(F + 1) * 4;
  if (e == cudaSuccess && order) e = cudaMemcpyAsync(order, ix.order, nb, cudaMemcpyDeviceToDevice, st);
  if (e == cudaSuccess && slot_of) e = cudaMemcpyAsync(slot_of, ix.slot_of, nb, cudaMemcpyDeviceToDevice, st);
  if (e == cudaSuccess && seg_begin) e = cudaMemcpyAsync(seg_begin, ix.seg_begin, fb, cudaMemcpyDeviceToDevice, st);
  if (e == cudaSuccess && item_begin) e = cudaMemcpyAsync(item_begin, ix.item_begin, fb, cudaMemcpyDeviceToDevice, st);
  if (e != cudaSuccess) return fail((int)e, "sort launches failed: %s", cudaGetErrorString(e));
  return 0;
}

size_t flexsae_index_skew_workspace_bytes(int64_t F) {
  if (F < 1 || F > (1ll << 30)) {
    fail(FLEXSAE_EINVAL, "F = %lld decoder rows outside the supported range", (long long)F);
    return 0;
  }
  return align_up((size_t)F * 4, 256);
}

int flexsae_index_skew(const int64_t* indices, int64_t B, int64_t K, int64_t F, void* workspace, size_t workspace_bytes,
                       int32_t* result, void* stream) {
  t_launches = 0;
  if (B < 1 || K < 1 || F < 1 || F > (1ll << 30) || B > (1ll << 40) / K)
    return fail(FLEXSAE_EINVAL, "B = %lld, K = %lld, F = %lld outside the supported range", (long long)B, (long long)K, (long long)F);
  if (!indices || !workspace || !result) return fail(FLEXSAE_EINVAL, "null pointer argument");
  const size_t need = align_up((size_t)F * 4, 256);
  if (workspace_bytes < need) return fail(FLEXSAE_EWORKSPACE, "skew workspace too small: %zu < %zu bytes", workspace_bytes, need);
  const long long n = (long long)B * K;
  long long stride = n / kSkewSamples;
  if (stride < 1) stride = 1;
  stride |= 1;  // odd: with K a power of two the samples then visit every one of the K columns
  const int samples = (int)((n + stride - 1) / stride < kSkewSamples ? (n + stride - 1) / stride : kSkewSamples);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(workspace, 0, (size_t)F * 4, st);
  if (e == cudaSuccess) e = cudaMemsetAsync(result, 0, 8, st);
  if (e == cudaSuccess) {
    index_skew_kernel<<<(samples + kSkewThreads - 1) / kSkewThreads, kSkewThreads, 0, st>>>(
        reinterpret_cast<const long long*>(indices), n, stride, samples, (int)F, reinterpret_cast<int*>(workspace), result);
    ++t_launches;
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) return fail((int)e, "skew launch failed: %s", cudaGetErrorString(e));
  return 0;
}

int flexsae_shard_slots(int64_t F, int64_t D, int weight_dtype) {
  Shape s{1, 1, F, D};
  if (check_shape(FLEXSAE_HIER, s, weight_dtype)) return 0;
  return plan_bwd(s, weight_dtype, FLEXSAE_DW_ATOMIC, true).pieces + kMaxSlabs + 1;  // an upper bound of the launch's slots for any lag
}

// ---- forward for callers that cannot provide scratch memory ------------------------------------
// The per-(piece, row) partial losses of the forward normally live in caller memory.  Here they
// live in a fixed array inside the library image: every GPU that loads the library carries these
// bytes until the process exits.
#define FLEXSAE_STATIC_PARTIALS (1u << 18) /* floats: 1 MiB */
static __device__ __align__(256) float g_static_loss_partials[FLEXSAE_STATIC_PARTIALS];

static std::mutex g_static_mutex;
static float* g_static_partials_addr[64];  // device ordinal -> device address of the array above

int flexsae_loss_fwd_static_scratch(int kind, const int64_t* indices, const void* weight, const void* vals,
                                    const void* bias, const void* target, float* loss_out, float* state_out,
                                    int segments, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype,
                                    int vals_dtype, int bias_dtype, int target_dtype, double inv_norm,
                                    int32_t* status, void* stream) {
  Shape s{B, K, F, D};
  if (int rc = check_shape(kind, s, weight_dtype)) return rc;
  const size_t need = plan_fwd(s, weight_dtype).total;
  const size_t have = sizeof(float) * FLEXSAE_STATIC_PARTIALS;
  if (need > have)
    return fail(FLEXSAE_EUNSUPPORTED,
                "the built-in scratch holds %zu bytes but this shape needs %zu (column pieces x B = %lld partial "
                "sums; at most %u): use flexsae_loss_fwd with caller memory",
                have, need, (long long)(need / sizeof(float)), (unsigned)FLEXSAE_STATIC_PARTIALS);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail((int)e, "cudaGetDevice failed: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(FLEXSAE_EUNSUPPORTED, "device ordinal %d outside [0, 64)", dev);
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_partials_addr[dev]) {
      // In host code the array's name is only a handle; the address the kernels need is asked
      // from the runtime once per device, with that device current.
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_loss_partials);
      if (e != cudaSuccess) return fail((int)e, "cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      g_static_partials_addr[dev] = reinterpret_cast<float*>(p);
    }
    scratch = g_static_partials_addr[dev];
  }
  // Every partial the final sum reads is written by this call's forward kernel first, so nothing
  // left over from an earlier call is ever read and nothing needs clearing.
  return flexsae_loss_fwd(kind, indices, weight, vals, bias, target, loss_out, state_out, segments, scratch, have, B, K,
                          F, D, weight_dtype, vals_dtype, bias_dtype, target_dtype, inv_norm, status, stream);
}

}  // extern "C"
