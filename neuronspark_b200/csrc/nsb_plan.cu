// Launch planner of the scan kernels: lanes per thread, warps per CTA, ring depth.
//
// The model behind the choice, from measurements on B200 (bf16, 196 608 columns,
// T = 8192): (1) the scan is bound by HBM bandwidth, so CTAs that are resident
// together share it and finish together; a launch may therefore run in several
// "waves" at no cost as long as every wave keeps enough bytes in flight; (2) a
// wave can never finish faster than one warp walks its T steps (about 100+70*V
// cycles per step forward, 1.4x that backward), which is what bounds problems
// with few columns and makes a small last wave expensive; (3) the bandwidth a
// pipeline reaches grows with the bytes moved per TMA tile (512 B: ~0.5 of peak,
// 1 KB: ~0.78, 2 KB: ~0.92, >= 4 KB: ~1). The cost of a candidate is the sum over
// its waves of max(bandwidth time, latency time, issue time) in microseconds.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <mutex>

#include "nsb_scan.cuh"

namespace nsb {

DeviceInfo b200_device_info() {
  DeviceInfo d;
  d.device = -1;
  d.sm_count = 148;
  d.cc_major = 10;
  d.cc_minor = 0;
  d.max_smem_optin = 232448;       // 227 KB per CTA
  d.smem_per_sm = 233472;          // 228 KB per SM
  d.reserved_smem_per_cta = 1024;
  return d;
}

namespace {

// Registers per thread of the kernel family (upper estimates from ptxas -v; they
// only bound how many warps fit an SM).
int regs_estimate(bool backward, int lanes, int tile, int modulated) {
  if (modulated) {  // scans with the modulation fused in: 1 = first order, 2 = resonate-and-fire
    const bool rf = modulated == 2;
    if (!backward) {
      if (lanes == 4) return rf ? 160 : 152;  // (the bit-packing variants need ~24 more; the launcher shrinks the CTA if so)
      if (lanes == 2) return rf ? 160 : 128;
      return tile == 32 ? (rf ? 168 : 96) : (rf ? 80 : 56);
    }
    if (lanes >= 2) return rf ? 136 : 104;
    return tile == 32 ? (rf ? 168 : 152) : (rf ? 80 : 64);
  }
  if (!backward) return lanes == 4 ? 72 : (lanes == 2 ? 56 : 48);
  if (tile * lanes <= 16) return 96;
  if (lanes == 1) return tile == 16 ? 128 : 200;
  return lanes == 4 ? 232 : 240;
}

double op_size_factor(double tile_bytes) {
  // bandwidth fraction reached as a function of bytes per TMA tile
  if (tile_bytes >= 4096.0) return 1.0;
  if (tile_bytes <= 256.0) return 0.3;
  const double pts_x[] = {256.0, 512.0, 1024.0, 2048.0, 4096.0};
  const double pts_y[] = {0.30, 0.50, 0.74, 0.92, 1.0};
  for (int i = 0; i < 4; ++i) {
    if (tile_bytes <= pts_x[i + 1]) {
      const double t = (std::log2(tile_bytes) - std::log2(pts_x[i])) /
                       (std::log2(pts_x[i + 1]) - std::log2(pts_x[i]));
      return pts_y[i] + t * (pts_y[i + 1] - pts_y[i]);
    }
  }
  return 1.0;
}

}  // namespace

Plan plan_scan(const DeviceInfo& d, const PlanQuery& q, const Tuning& tune) {
  Plan best;
  best.grid = 0;
  double best_cost = 1e300;
  const int sms = std::max(1, d.sm_count);
  const int reserved = d.reserved_smem_per_cta > 0 ? d.reserved_smem_per_cta : 1024;
  const int ntiles = (int)((q.T + q.tile - 1) / q.tile);
  // Plain forward scans over many columns (a full chip's worth of 4-lane warps and more): measured
  // over 196 K .. 6.3 M columns the wave model below misjudges them (it once chose 7-warp CTAs for
  // 786 K columns: 0.87 of the HBM peak where 2- and 4-warp CTAs reach 0.98), while one shape is
  // within 2 % of the best everywhere: long scans, 4 lanes x 4 warps x 2 stages; scans of a few
  // tiles (per-token decoding), where CTA start-up dominates, 1- or 2-warp CTAs with 4 lanes per
  // thread from 1.5 M columns on and 2 below.
  // (The plain row-parameter scan, 1 stream, long: 196 608 columns 1.22 ms with this shape against 1.53.)
  if (!q.backward && !q.modulated && q.stash == 0 && q.tile == 8 && q.max_lanes >= 4 && q.cols >= 196608 &&
      (q.nstreams >= 3 || (q.nstreams == 1 && ntiles > 8)) &&
      tune.warps_per_cta <= 0 && tune.stages <= 0 && tune.lanes_per_thread <= 0) {
    const bool few_tiles = ntiles <= 8;
    const int lanes = (few_tiles && q.cols < 1500000) ? 2 : 4;
    const int wpc = few_tiles ? (lanes == 4 ? 1 : 2) : 4;
    const size_t stage_bytes = (size_t)q.tile * 32 * lanes * q.elem_size * q.nstreams;
    const size_t smem = (size_t)wpc * 2 * (stage_bytes + 8) + 256;
    if (smem + reserved <= (size_t)d.smem_per_sm / 2) {
      const long long nwarps = (q.cols + 32LL * lanes - 1) / (32LL * lanes);
      best.lanes = lanes;
      best.wpc = wpc;
      best.stages = 2;
      best.grid = (int)((nwarps + wpc - 1) / wpc);
      best.smem = smem;
      best.cost = 0.0;
      return best;
    }
  }
  // Row-parameter backward (the drive and the incoming gradient: 2 streams) over many columns: 4 lanes
  // in 2-warp CTAs with a 3-deep ring, measured at T = 8192, bf16: 147 456 columns 1.37 ms against 1.49
  // for the 2-lane shapes chosen below, 196 608 columns 1.78 against 2.14.
  if (q.backward && !q.modulated && q.stash == 0 && q.tile == 8 && q.max_lanes >= 4 && q.nstreams <= 2 &&
      q.cols >= 147456 && ntiles > 8 && tune.warps_per_cta <= 0 && tune.stages <= 0 && tune.lanes_per_thread <= 0) {
    const int lanes = 4, wpc = 2, st = 3;
    const size_t stage_bytes = (size_t)q.tile * 32 * lanes * q.elem_size * q.nstreams;
    const size_t smem = (size_t)wpc * st * (stage_bytes + 8) + 256;
    if (smem + reserved <= (size_t)d.smem_per_sm / 2) {
      const long long nwarps = (q.cols + 32LL * lanes - 1) / (32LL * lanes);
      best.lanes = lanes;
      best.wpc = wpc;
      best.stages = st;
      best.grid = (int)((nwarps + wpc - 1) / wpc);
      best.smem = smem;
      best.cost = 0.0;
      return best;
    }
  }
  // Calibration constants (B200): HBM bytes per microsecond, SM clock in cycles per
  // microsecond, time from CTA start until its first tile has landed.
  const double hbm_bytes_per_us = 6.5e6, clk_per_us = 1.9e3, t_start_us = 4.0;
  // HBM bytes per neuron-step: the streamed inputs plus the outputs written back
  // (dense forward: spikes; backward: one gradient per forward input).
  const double bytes_per_ns = q.elem_size * (q.backward ? (2.0 * q.nstreams - 1.0) : (q.nstreams + 1.0));
  const int lane_opts[3] = {4, 2, 1};
  for (int lanes : lane_opts) {
    if (lanes > q.max_lanes) continue;
    if (tune.lanes_per_thread > 0 && lanes != tune.lanes_per_thread) continue;
    // Scans of a few tiles only (per-token decoding) are dominated by CTA start-up;
    // measured: 2 lanes per thread (twice the CTAs per SM) beat 4 by ~20 % at T = 16.
    if (tune.lanes_per_thread <= 0 && ntiles <= 8 && lanes > 2) continue;
    // 16-step tiles of the selective / resonate-and-fire scans over 32 K columns and more: 2 lanes per
    // thread (measured at 49 152 columns, T = 8192, bf16: forward 649 us against 742 with 1 lane,
    // forward + backward 2.16 ms against 2.27)
    if (tune.lanes_per_thread <= 0 && q.tile == 16 && q.nstreams >= 3 && q.cols >= 32768 && q.max_lanes >= 2 &&
        lanes != 2)
      continue;
    const long long nwarps = (q.cols + 32LL * lanes - 1) / (32LL * lanes);
    const size_t tile_bytes = (size_t)q.tile * 32 * lanes * q.elem_size;
    const size_t stage_bytes = tile_bytes * q.nstreams;
    const int regs = regs_estimate(q.backward, lanes, q.tile, q.modulated);
    // each of the 4 SM sub-partitions has its own 16 K registers and takes every 4th warp
    const int reg_warps = std::max(1, 4 * (16384 / (regs * 32)));
    const double f_op = op_size_factor((double)tile_bytes);
    // A lone warp advances one time step in about this many cycles (dependent
    // chain + per-tile overheads), and needs about this many issue slots for it.
    const double cyc_per_step = (q.backward ? 1.4 : 1.0) * (100.0 + 70.0 * lanes);
    const double issue_per_step = (q.backward ? 2.0 : 1.0) * (20.0 + 15.0 * lanes);
    for (int wpc = 1; wpc <= 16; ++wpc) {
      if (tune.warps_per_cta > 0 && wpc != tune.warps_per_cta) continue;
      for (int st = 2; st <= 6; ++st) {
        if (tune.stages > 0 && st != tune.stages) continue;
        if (tune.stages <= 0 && (st > 4 || st > std::max(2, ntiles))) continue;
        const int stash = (lanes == 2 && q.stash_2lanes >= 0) ? q.stash_2lanes : q.stash;
        const size_t smem = (size_t)wpc * (st * (stage_bytes + 8) + (size_t)stash * q.tile * 32 * lanes * 4) + 256;
        if (smem > (size_t)d.max_smem_optin) continue;
        long long res = std::min<long long>(32, d.smem_per_sm / (long long)(smem + reserved));
        res = std::min<long long>(res, 64 / wpc);
        res = std::min<long long>(res, reg_warps / wpc);
        if (res < 1) continue;
        const long long ctas = (nwarps + wpc - 1) / wpc;
        const long long cap = res * sms;
        double cost = 0.0;  // microseconds
        long long remaining = ctas;
        while (remaining > 0) {
          const long long w = std::min(cap, remaining);
          const double warps = (double)w * wpc;
          const double t_bw = warps * 32.0 * lanes * (double)q.T * bytes_per_ns / (hbm_bytes_per_us * f_op);
          const double t_lat = t_start_us + (double)q.T * cyc_per_step / clk_per_us;
          const double warps_per_sched = std::max(1.0, warps / (sms * 4.0));
          const double t_issue = warps_per_sched * (double)q.T * issue_per_step / clk_per_us;
          const double t_wave = std::max(t_bw, std::max(t_lat, t_issue));
          if (ctas > 8 * cap) {  // many waves: they all look like this one
            cost = t_wave * (double)ctas / (double)w;
            break;
          }
          cost += t_wave;
          remaining -= w;
        }
        // Near-ties: more resident columns per SM hide more latency (measured on the
        // bit-packed forward: 13 resident warps of 4 lanes beat 8 by 30 %); then a 3-deep
        // ring over a 2-deep one, then small CTAs.
        const double resident_lanes = (double)std::min(cap, ctas) * wpc * 32.0 * lanes / sms;
        cost *= 1.0 + 0.03 * std::max(0.0, 1.0 - resident_lanes / 1536.0);
        cost *= 1.0 + 0.004 * std::abs(st - 3) + 0.002 * wpc;
        if (cost < best_cost) {
          best_cost = cost;
          best.lanes = lanes;
          best.wpc = wpc;
          best.stages = st;
          best.grid = (int)ctas;
          best.smem = smem;
          best.cost = cost;
        }
      }
    }
  }
  return best;
}

// ---- time split of forward scans over few columns
//
// A scan over a few thousand columns keeps a few hundred warps busy while the chip has 592 warp
// schedulers, and each warp is bound by its own serial chain over T. Spare schedulers can take
// later parts of the time axis: a segment is entered `warm` steps early from V = 0, and by its
// own first step its state equals the exact one bit for bit (two PLIF trajectories driven by the
// same input merge once their difference has decayed below one unit in the last place: within
// 200-650 steps for the benchmark distributions, measured on CPU). A second launch verifies this
// per column and rescans what differs, so the result is exact whatever the inputs.
namespace {
std::atomic<int> g_split_max_segments{0};  // 0 = automatic, 1 = never split
std::atomic<int> g_split_warm_steps{0};    // 0 = default
thread_local TimeSplit g_last_split;
constexpr int kDefaultWarmSteps = 1024;
constexpr int kMaxSegments = 16;
constexpr long long kSplitMaxCols = 37888;  // four warps per scheduler and two segments
}  // namespace

TimeSplit& last_time_split() { return g_last_split; }

// The backward keeps 4 rows per segment. Scans over more columns than the split ever takes (four warps per
// scheduler and two segments: 37 888 columns) need only the counters of a chained backward launch.
long long time_split_scratch_floats(long long cols) {
  if (cols <= 0) return 0;
  const long long split = cols <= kSplitMaxCols ? 4LL * kMaxSegments * cols + 4 : 0;
  return std::max(split, chain_scratch_words(cols));
}

TimeSplit plan_time_split(const DeviceInfo& dev, long long T, long long cols, int tile, int lanes, int wpc,
                          bool backward, int family) {
  TimeSplit ts;
  const int cap = g_split_max_segments.load(std::memory_order_relaxed);
  if (cap == 1 || tile <= 0 || cols > kSplitMaxCols) return ts;
  // The scans of the layers' hidden neurons forget as slowly as their largest beta lets them (0.99 at the
  // reference's initialisation: 1 650 steps to lose 24 bits), and a resonate-and-fire column whose
  // beta^2 + omega^2 sits at the stability clamp contracts by 0.999 a step: a 1 024-step warm-up then
  // leaves segments to rescan, and one rescanned segment undoes the gain. Measured, forward at T = 8192,
  // 6 144 columns: resonate-and-fire 313 -> 142 us with 6 segments, first order with the modulation 561 ->
  // 288 us with 4, both without a rescan on short-memory parameters; resonate-and-fire with the modulation
  // 892 -> 945-1000 us because 1-3 % of the warps rescanned. So these split only where the caller, who
  // knows the dynamics, asks for it.
  if (family != 0 && cap <= 1) return ts;
  const long long ntiles = (T + tile - 1) / tile;
  const long long nwarps = (cols + 32LL * lanes - 1) / (32LL * lanes);
  const long long ctas = (nwarps + wpc - 1) / wpc;
  // Up to four warps per scheduler. A scheduler with several warps of this chain-bound code advances each
  // of them more slowly than a lone one, but more segments still win while the product falls. Measured at
  // T = 8192, ns per step and warp with 1 / 2 / 3 / 4 warps on the busiest scheduler: forward 27 / 33 / 38 /
  // 45, backward 38 / 52 / 65 / 95 (384 and 768 column warps cut into 1-6 segments). Examples: 6 144 columns
  // forward 114 us with 3 segments (one warp per scheduler), 83 with 6; backward 157 -> 139 us; 12 288 columns,
  // which one warp per scheduler cannot split, forward 220 -> 109 us (6 segments), backward 313 -> 198 (3);
  // 24 576 columns forward 239 -> 171 us (3), backward 417 -> 313 (2). The slowest scheduler sets the time,
  // so the factor goes by the rounded-up number of warps per scheduler.
  const long long schedulers = 4LL * std::max(1, dev.sm_count);
  static const double kFwd[5] = {1.0, 1.0, 1.23, 1.41, 1.68}, kBwd[5] = {1.0, 1.0, 1.37, 1.7, 2.5};
  auto crowd = [&](long long warps) {
    const long long w = std::min<long long>(4, std::max<long long>(1, (warps + schedulers - 1) / schedulers));
    return backward ? kBwd[w] : kFwd[w];
  };
  long long pmax = 4 * schedulers / std::max(1LL, ctas * wpc);
  pmax = std::min<long long>(pmax, cap > 1 ? cap : kMaxSegments);
  pmax = std::min<long long>(pmax, kMaxSegments);
  const int warm_steps = g_split_warm_steps.load(std::memory_order_relaxed);
  const long long warm = ((warm_steps > 0 ? warm_steps : kDefaultWarmSteps) + tile - 1) / tile;
  long long best_p = 1;
  const double unsplit_cost = (double)ntiles * crowd(ctas * wpc);
  double best_cost = unsplit_cost;
  for (long long pseg = 2; pseg <= pmax; ++pseg) {
    const long long seg = (ntiles + pseg - 1) / pseg;
    if (seg < warm || seg * (pseg - 1) >= ntiles) continue;  // warm-up would reach before t = 0 / an empty last segment
    const double cost = (double)(seg + warm) * crowd(ctas * wpc * pseg);
    if (cost < best_cost) {
      best_cost = cost;
      best_p = pseg;
    }
  }
  // worth two launches only if a tenth of the time goes away (an explicit cap > 1 is obeyed as is; 36 864
  // columns, predicted 0.85: forward 270 -> 230 us)
  if (best_p > 1 && (cap > 1 || best_cost <= 0.9 * unsplit_cost)) {
    ts.nseg = (int)best_p;
    ts.seg_tiles = (int)((ntiles + best_p - 1) / best_p);
    ts.warm_tiles = (int)warm;
    // the second launch lasts as long as its busiest warp rescans, at a lone warp's pace
    ts.allow_rescans = (int)std::max(0.0, std::floor((unsplit_cost - best_cost) / (double)ts.seg_tiles));
  }
  return ts;
}

// ---- what split launches had to rescan, fed back
//
// The split pays while segments merge with the exact trajectory inside the warm-up. A neuron trained
// to a long memory (beta near 1) does not, and then the two launches cost more than the plain scan.
// Each automatic split launch therefore copies its two counter words to pinned host memory, and the
// next launch for the same neuron reads them - whatever has arrived by then, without waiting: if one
// warp had to rescan more segments than the split saved, that neuron's scans go unsplit for the next
// 64 calls and then try again.
namespace {
struct FeedbackEntry {
  const void* neuron;
  long long T, cols;
  int backward, allow, skip_left;
};
constexpr int kFeedbackSlots = 256;
constexpr int kBackoffCalls = 64;
FeedbackEntry g_fb[kFeedbackSlots];
int g_fb_used = 0, g_fb_next = 0;
unsigned int* g_fb_host = nullptr;  // pinned, two words per slot
bool g_fb_failed = false;
std::mutex g_fb_mu;

int feedback_find(const void* neuron, long long T, long long cols, bool backward) {
  for (int i = 0; i < g_fb_used; ++i)
    if (g_fb[i].neuron == neuron && g_fb[i].T == T && g_fb[i].cols == cols && g_fb[i].backward == (int)backward) return i;
  return -1;
}
}  // namespace

bool time_split_automatic() { return g_split_max_segments.load(std::memory_order_relaxed) == 0; }

bool split_feedback_allows(const void* neuron, long long T, long long cols, bool backward) {
  std::lock_guard<std::mutex> lk(g_fb_mu);
  const int i = feedback_find(neuron, T, cols, backward);
  if (i < 0 || !g_fb_host) return true;
  FeedbackEntry& e = g_fb[i];
  if (e.skip_left > 0) {
    --e.skip_left;
    return false;
  }
  volatile unsigned int* h = g_fb_host + 2 * i;
  if ((long long)h[1] > (long long)e.allow) {
    h[0] = h[1] = 0;
    e.skip_left = kBackoffCalls - 1;
    return false;
  }
  return true;
}

void split_feedback_record(const void* neuron, long long T, long long cols, bool backward,
                           const unsigned int* dev_words, int allow_rescans, cudaStream_t stream) {
  std::lock_guard<std::mutex> lk(g_fb_mu);
  if (g_fb_failed) return;
  if (!g_fb_host) {
    // (pinned memory cannot be allocated while the stream is being captured into a graph)
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone) {
      cudaGetLastError();
      return;
    }
    void* h = nullptr;
    if (cudaHostAlloc(&h, sizeof(unsigned int) * 2 * kFeedbackSlots, cudaHostAllocPortable) != cudaSuccess) {
      cudaGetLastError();  // no feedback then; the split stays exact, only its choice is blind
      g_fb_failed = true;
      return;
    }
    memset(h, 0, sizeof(unsigned int) * 2 * kFeedbackSlots);
    g_fb_host = static_cast<unsigned int*>(h);
  }
  int i = feedback_find(neuron, T, cols, backward);
  if (i < 0) {
    if (g_fb_used < kFeedbackSlots) {
      i = g_fb_used++;
    } else {  // oldest first
      i = g_fb_next;
      g_fb_next = (g_fb_next + 1) % kFeedbackSlots;
    }
    g_fb[i] = FeedbackEntry{neuron, T, cols, (int)backward, allow_rescans, 0};
    g_fb_host[2 * i] = g_fb_host[2 * i + 1] = 0;
  }
  g_fb[i].allow = allow_rescans;
  if (cudaMemcpyAsync(g_fb_host + 2 * i, dev_words, 2 * sizeof(unsigned int), cudaMemcpyDeviceToHost, stream) !=
      cudaSuccess)
    cudaGetLastError();
}

// ---- rotation of a forward scan with the modulation fused in
//
// With few columns there are too few warps for the issue slots: 49 152 columns of the resonate-and-fire
// scan with one lane per thread are 1 536 warps for 592 schedulers, each warp issuing one instruction
// every 4.6 cycles (56 % of the issue slots busy, special-function pipe 46 %, DRAM 44 %). Two thirds of
// those instructions - the modulation - do not depend on the membrane state, so R warps share a column
// group and take its tiles in turn; only the recurrence's own few instructions per step wait for the
// predecessor. R is chosen for about five warps per scheduler.
namespace {
std::atomic<int> g_rotation{0};  // 0 = automatic, 1 = never, 2..4 = that many warps per column group
thread_local int g_last_rotation = 1;
}  // namespace

int& last_rotation() { return g_last_rotation; }
bool get_rotation_forced() { return g_rotation.load(std::memory_order_relaxed) > 1; }

int plan_rotation(const DeviceInfo& dev, long long column_warps, int ntiles) {
  const int forced = g_rotation.load(std::memory_order_relaxed);
  if (forced == 1 || column_warps <= 0) return 1;
  long long r = forced;
  if (forced == 0) {
    const long long schedulers = 4LL * std::max(1, dev.sm_count);
    // Measured (resonate-and-fire, T = 8192, bf16, forward ms, one warp per group on 32-step tiles -> rotating
    // on 8-step tiles): 192 column warps 0.89 -> 0.50 (3 warps per group; 0.67 with 2, 0.51 with 4), 384:
    // 0.89 -> 0.57 (4), 768: 1.00 -> 0.88 (3; 0.90 with 2 or 4); first order 192: 0.62 -> 0.43. With 1 536
    // column warps (2.6 per scheduler already) two warps per group are a loss: 1.43 -> 1.80 ms.
    if (2 * column_warps > 3 * schedulers) return 1;
    r = (5 * schedulers + column_warps / 2) / column_warps;
  }
  r = std::min<long long>(4, std::max<long long>(1, r));
  while (r > 1 && ntiles < 4 * r) --r;  // every warp of a group gets a few tiles
  return (int)r;
}

// ---- chained chunks of a backward launch
//
// A backward launch over many columns has more CTAs than fit on the GPU at once, and a CTA walks all
// of T: with 768 CTAs for 444 places the second round is 73 % full and lasts as long as the first.
// Cut into q chunks of the time axis the launch has q times as many pieces of work of 1/q the
// length, handed out in time order, so the GPU stays full until the end - and all resident CTAs
// work on the same few rows of every [T, cols] tensor at any moment, which DRAM likes: the gain
// grows well beyond what the emptier last round explains. Measured (B200, bf16, T = 8192,
// 196 608 columns, 8-step tiles; backward ms for 1 / 4 / 8 / 16 / 32 / 64 / 128 / 256 chunks):
//   selective, gain*cur form   5.12 / 4.94 / 4.83 / 4.76 / 4.66 / 4.57 / 4.59 / 5.08
//   resonate-and-fire          5.26 /  -   / 4.95 / 4.88 / 4.78 / 4.74 / 4.82 /  -
//   first order + modulation   5.50 / 5.02 / 4.86 / 4.84 / 5.18* / 5.50* (* another box: 5.11 at 8)
//   resonate-and-fire + mod.   8.96 / 7.85 / 7.80 / 7.81 / 8.27 / 8.43 (6 chunks: 7.73)
// A chunk costs a pipeline start (ticket, first tiles' latency, and in the modulated kernels the
// per-channel biases), so the plain scans take chunks of 128 steps and the modulated ones of 1024.
// Launches that fit the GPU (same sizes, fewer columns; backward ms unchained / 16 / 64 chunks):
//   selective, 98 304 columns  2.99 / 2.46 / 2.36      49 152 columns  1.42 / 1.29 / 1.40
//   selective, 24 576 columns  0.69 / 0.71 / 0.89      linear recurrence, 196 608: 3.81 / 3.00 / 2.80 (128: 2.70)
//   modulated, 49 152 - 98 304 columns: no gain or a loss; row-parameter, 196 608: 2.14 / 2.17 / 2.45
// so plain scans are chained from 49 152 columns on (chunks of 512 steps below 98 304 columns), the
// modulated ones only where the launch exceeds the GPU, the row-parameter one only on request.
namespace {
std::atomic<int> g_chain_chunks{0};  // 0 = automatic, 1 = never, n = n chunks on every launch that has the scratch
std::atomic<int> g_last_chain{1};  // process-wide: the backward usually runs on a thread of the caller's autograd engine
constexpr int kMaxChainChunks = 1024;
constexpr int kMinChainTiles = 4;
}  // namespace

void set_last_chain_chunks(int q) { g_last_chain.store(q, std::memory_order_relaxed); }
int last_chain_chunks() { return g_last_chain.load(std::memory_order_relaxed); }

long long chain_scratch_words(long long cols) { return cols > 0 ? cols / 32 + 128 : 0; }

int plan_chain_chunks(bool eligible, int ntiles, int target_tiles) {
  const int forced = g_chain_chunks.load(std::memory_order_relaxed);
  if (forced > 1) return std::max(1, std::min(forced, ntiles));  // (whatever the launch)
  if (forced == 1 || !eligible) return 1;
  const int tiles = std::max(kMinChainTiles, target_tiles);
  const int q = std::min(kMaxChainChunks, ntiles / tiles);
  return q >= 2 ? q : 1;
}

}  // namespace nsb

extern "C" int nsb_set_scan_rotation(int warps) {
  if (warps < 0 || warps > 4) return NSB_ERR_INVALID_ARG;
  nsb::g_rotation.store(warps, std::memory_order_relaxed);
  return NSB_OK;
}
extern "C" int nsb_last_scan_rotation(void) { return nsb::last_rotation(); }
extern "C" int nsb_scan_rotation_query(int64_t T, int64_t cols, int tile) {
  if (T < 0 || cols <= 0 || tile <= 0) return 0;
  return nsb::plan_rotation(nsb::b200_device_info(), (cols + 31) / 32, (int)((T + tile - 1) / tile));
}

extern "C" int nsb_set_chain_chunks(int chunks) {
  if (chunks < 0 || chunks > 1024) return NSB_ERR_INVALID_ARG;
  nsb::g_chain_chunks.store(chunks, std::memory_order_relaxed);
  return NSB_OK;
}
extern "C" int nsb_last_chain_chunks(void) { return nsb::last_chain_chunks(); }
extern "C" int64_t nsb_chain_scratch_words(int64_t cols) { return nsb::chain_scratch_words(cols); }

extern "C" int nsb_set_time_split(int max_segments, int warm_steps) {
  if (max_segments < 0 || max_segments > 16 || warm_steps < 0) return NSB_ERR_INVALID_ARG;
  nsb::g_split_max_segments.store(max_segments, std::memory_order_relaxed);
  nsb::g_split_warm_steps.store(warm_steps, std::memory_order_relaxed);
  {  // a new setting starts without memory of what earlier launches rescanned
    std::lock_guard<std::mutex> lk(nsb::g_fb_mu);
    nsb::g_fb_used = nsb::g_fb_next = 0;
  }
  return NSB_OK;
}

extern "C" int64_t nsb_time_split_scratch_floats(int64_t cols) {
  return cols > 0 ? nsb::time_split_scratch_floats(cols) : 0;
}

extern "C" int nsb_last_time_split(int32_t out[3]) {
  if (!out) return NSB_ERR_INVALID_ARG;
  const nsb::TimeSplit& ts = nsb::last_time_split();
  out[0] = ts.nseg;
  out[1] = ts.seg_tiles;
  out[2] = ts.warm_tiles;
  return NSB_OK;
}

extern "C" int nsb_time_plan_query(int backward, int modulated, int64_t T, int64_t cols, int tile, int lanes,
                                   int warps_per_cta, int32_t out[4]) {
  if (!out || T < 0 || cols <= 0 || (tile != 8 && tile != 16 && tile != 32) || lanes < 1 || lanes > 4 ||
      warps_per_cta < 1 || warps_per_cta > 32)
    return NSB_ERR_INVALID_ARG;
  const nsb::TimeSplit ts = nsb::plan_time_split(nsb::b200_device_info(), T, cols, tile, lanes, warps_per_cta,
                                                 backward != 0, modulated ? 2 : 0);
  out[0] = ts.nseg;
  out[1] = ts.seg_tiles;
  out[2] = ts.warm_tiles;
  // chained chunks a backward launch over these columns would take (selective / resonate-and-fire / linear
  // scans by their width; with the modulation fused in, where the launch exceeds the GPU: 444 places of 4 warps)
  const int ntiles = (int)((T + tile - 1) / tile);
  const long long warps = (cols + 32LL * lanes - 1) / (32LL * lanes);
  const bool eligible = modulated ? (warps + warps_per_cta - 1) / warps_per_cta > 3LL * nsb::b200_device_info().sm_count
                                  : cols >= 49152;
  out[3] = backward ? nsb::plan_chain_chunks(eligible, ntiles, (modulated ? 1024 : (cols >= 98304 ? 128 : 512)) / tile) : 1;
  return NSB_OK;
}

extern "C" int nsb_scan_plan_query(int backward, int nstreams, int elem_size, int64_t T, int64_t cols,
                                   int tile, int32_t out[5]) {
  if (!out || T < 0 || cols <= 0 || nstreams < 1 || nstreams > 6 || (elem_size != 2 && elem_size != 4) ||
      (tile != 8 && tile != 16 && tile != 32))
    return NSB_ERR_INVALID_ARG;
  nsb::PlanQuery q;
  q.T = T;
  q.cols = cols;
  q.elem_size = elem_size;
  q.nstreams = nstreams;
  q.tile = tile;
  q.backward = backward != 0;
  q.max_lanes = tile == 32 ? 1 : ((backward && tile == 16) ? 2 : 4);
  const nsb::Plan p = nsb::plan_scan(nsb::b200_device_info(), q, nsb::get_tuning());
  if (p.grid == 0) return NSB_ERR_UNSUPPORTED;
  out[0] = p.lanes;
  out[1] = p.wpc;
  out[2] = p.stages;
  out[3] = p.grid;
  out[4] = (int32_t)p.smem;
  return NSB_OK;
}
