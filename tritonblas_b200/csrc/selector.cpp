// Analytical tile / schedule selector for B200, the native counterpart of the reference's external `origami`
// model (call sites include/tritonblas/origami.py:166,232-262) and of its stream-K grid rule (:349-416).
//
// The model is derived for the machine, not transcribed: a CTA owns 128 accumulator rows (TMEM lanes) and a tile
// width BN in {32..256}; two CTAs of a cluster may pair up on a 256 x BN tile so each stages only half of B. Every
// shared-memory stage holds 128 bytes of K per operand row, so for every operand type one stage costs
//     mma clocks   = 2 * BN                      (4 MMAs of 128 x BN x 32 bytes-of-K, BN/2 clocks each)
//     fill bytes   = (128 + BN / pair) * 128     (this CTA's A rows + its share of B rows)
// and a tile costs num_k_blocks * max(mma, fill / fabric bytes-per-clock) clocks. A data-parallel launch runs
// ceil(tiles / programs) waves of that; a stream-K launch runs tiles * num_k_blocks / programs stages per program
// plus the fix-up of one partial tile. Whole-problem HBM time is a floor under both.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>

#include "../../include/tritonblas_b200.h"
#include "selector.h"

namespace tb {

static int esize_of(int dtype) {
  switch (dtype) {
    case TB_DTYPE_F16:
    case TB_DTYPE_BF16: return 2;
    case TB_DTYPE_F32: return 4;
    case TB_DTYPE_E4M3:
    case TB_DTYPE_E5M2:
    case TB_DTYPE_I8:
    case TB_DTYPE_U8: return 1;
    default: return 0;
  }
}

static int next_pow2(int v) {
  int r = 32;
  while (r < v) r <<= 1;
  return r;
}

int smem_bytes_for(int block_n, int cta_pair, int stages, int n_halves) {
  const int stage = 128 * 128 + n_halves * (block_n / cta_pair) * 128;
  return stages * stage + 16384 + (2 * stages + 16) * 8 + 64 + 1024;  // ring + epilogue staging + barriers + tile queue + slots + slack
}

struct Candidate {
  int bn, pair, halves;
  double dp_us, sk_us;
  int grid, sk_grid, stages, group_m;
};

int select_config(const tb_problem& p_in, const MachineModel& hw, tb_config* out) {
  if (p_in.m <= 0 || p_in.n <= 0 || p_in.k <= 0) return TB_ERR_INVALID;
  const bool mx = p_in.mx_block_size == 32 || p_in.a_dtype == TB_DTYPE_F4;
  // Few rows of A against a wide B (decode shapes): compute C^T = B^T A^T so the streamed matrix fills the 128-row side
  // of the tile and the few rows become a narrow tile width; shared memory then holds almost only streamed data.
  tb_problem p = p_in;
  const bool swap = !mx && p_in.m <= 64 && p_in.n >= 256 && p_in.n >= 4 * p_in.m;
  if (swap) {
    p.m = p_in.n;
    p.n = p_in.m;
    p.a_mn_major = p_in.b_mn_major;
    p.b_mn_major = p_in.a_mn_major;
  }
  const int es = mx ? 1 : esize_of(p.a_dtype);
  if (es == 0) return TB_ERR_UNSUPPORTED;
  const int sms = (p.num_sms > 0 && p.num_sms <= hw.num_sms) ? p.num_sms : hw.num_sms;
  // K elements per stage: 128 bytes of K; packed fp4 carries two elements per byte.
  const int bk = mx ? 256 : 128 / es;
  const int nkb = (p.k + bk - 1) / bk;
  const int mn_atom = 128 / es;  // an N-contiguous B is staged in boxes of this many columns
  const double c_bytes = static_cast<double>(p.m) * p.n * esize_of(p.c_dtype);
  const double ab_bytes = (static_cast<double>(p.m) * p.k + static_cast<double>(p.n) * p.k) * (mx ? 0.5 : es);
  const double hbm_us = (c_bytes + ab_bytes) / (hw.hbm_gbs * 1e3);
  // fp4 MMAs retire 64 bytes of K per instruction at the clocks an 8/16-bit MMA needs for 32.
  const double mma_clk_per_stage_per_bn = mx ? 1.0 : 2.0;

  Candidate best{};
  double best_cost = 1e30;
  // Block-scaled kinds keep their scale factors in TMEM beside two accumulator stages and need tile starts that are
  // multiples of 64 columns, which leaves 192, 128 and 64.
  static const int kBNDense[] = {256, 128, 64, 32, 0};
  static const int kBNMx[] = {192, 128, 64, 0};
  const int* widths = mx ? kBNMx : kBNDense;
  for (int pair = 2; pair >= 1; --pair) {
    if (pair == 2 && (sms < 2 || !hw.allow_pair)) continue;
    // A pair halves each CTA's share of B; with at most 128 rows of A the second CTA of a pair would only multiply
    // padding, and partial tiles of a stream-K launch would double in size.
    if (pair == 2 && (p.m <= 128 || p.n <= 64)) continue;
    for (int wi = 0; widths[wi] != 0; ++wi) {
      const int bn = widths[wi];
      const int bn_local = bn / pair;
      if (p.b_mn_major && (bn_local % mn_atom) != 0) continue;
      if (bn >= 2 * p.n && bn > 32 && !(p.b_mn_major && bn <= mn_atom)) continue;  // more than half the tile would be padding
      if (bn_local < 16) continue;
      // A wide tile (two bn-wide accumulators that share every A stage) only pays at the full accumulator width, and
      // the stream-K, block-scaled and grouped paths do not take it.
      const int max_halves = (!mx && !p.streamk && p.max_halves != 1 && bn == 256 && p.n >= 2 * bn) ? 2 : 1;
      for (int halves = max_halves; halves >= 1; --halves) {
      const int tile_m = 128 * pair;
      const int tile_n = bn * halves;
      const long long tiles_m = (p.m + tile_m - 1) / tile_m, tiles_n = (p.n + tile_n - 1) / tile_n;
      const long long tiles = tiles_m * tiles_n;
      const int programs = std::max(1, sms / pair);
      const int sf_bytes = mx ? (2 + 2 * 2) * 512 : 0;
      const int stage_bytes = (128 * 128 + halves * bn_local * 128 + sf_bytes + 1023) & ~1023;
      int stages = (hw.smem_optin - 2048 - 16384) / stage_bytes;
      stages = std::min(stages, 12);
      // Transposed (decode) orientation: the launch is bound by the rate at which one SM pulls its rows out of HBM, and
      // that rate peaks with about 160 KB requested ahead (measured on 16 x 28672 x 8192 bf16: 3 / 4 / 6 / 8 / 10 stages
      // of 20 KB: 98.9 / 91.6 / 87.8 / 86.8 / 89.3 us; 64-column tiles: best at 6-7 stages of 24 KB).
      if (swap) stages = std::min(stages, std::max(4, 168 * 1024 / stage_bytes));
      if (stages < 2) continue;
      const long long active_ctas = std::min<long long>(tiles, programs) * pair;
      // L2 -> shared memory: one SM alone pulls fabric_bytes_per_clk, all of them together share the L2's total
      const double fabric = std::min(hw.fabric_bytes_per_clk, hw.l2_bytes_per_clk / static_cast<double>(active_ctas));
      const double mma_clk = mma_clk_per_stage_per_bn * bn * halves;
      const double fill_clk = (128.0 + halves * bn_local) * 128.0 / fabric;
      // Measured: with narrow tiles every MN-major operand costs about 10-15 % (8192^2 x 4096 bf16: 1260 / 1155 / 1021
      // TFLOP/s for 0 / 1 / 2 such operands), with wide tiles nothing (1272 / 1276 / 1257).
      const double mn_penalty = halves == 1 ? 1.0 + 0.15 * ((p.a_mn_major ? 1 : 0) + (p.b_mn_major ? 1 : 0)) : 1.0;
      const double stage_clk = std::max(mma_clk, fill_clk) * mn_penalty;
      const double ramp_clk = hw.tile_ramp_clk;  // first-stage latency + epilogue drain not hidden by the next tile
      const double clk_to_us = 1.0 / (hw.sm_mhz);
      // Draining one 128 x bn accumulator. Two accumulator stages hide it behind the next tile's main loop unless
      // that loop is shorter; a wide tile owns both stages, so its two drains are exposed.
      const double drain_clk = 1000.0 + 12.0 * bn;
      // HBM floor: one SM cannot pull its share of the full bandwidth alone, so idle SMs cost bandwidth
      auto hbm_floor = [&](long long active) {
        const double share = std::min(1.0, 1.15 * static_cast<double>(active) / hw.num_sms);
        return hbm_us / share;
      };
      // data-parallel
      const long long waves = (tiles + programs - 1) / programs;
      const double tile_clk = halves == 2 ? nkb * stage_clk + 2.0 * drain_clk : std::max(nkb * stage_clk, drain_clk);
      double dp = (waves * tile_clk + ramp_clk + drain_clk) * clk_to_us;
      // HBM floor per wave: the bytes of the full waves move with every program pulling, those of the ragged last wave
      // with only its programs pulling (224 tiles on 148 programs: the last 76 tiles stream at 0.59 of the bandwidth).
      {
        const long long full = tiles / programs, rem = tiles % programs;
        double floor_us = 0.0;
        if (full > 0) floor_us += hbm_floor(static_cast<long long>(programs) * pair) * (static_cast<double>(full * programs) / tiles);
        if (rem > 0) floor_us += hbm_floor(rem * pair) * (static_cast<double>(rem) / tiles);
        dp = std::max(dp, floor_us) + hw.launch_us;
      }
      // stream-K: stages per program, plus one partial tile written and read back through L2, plus the flag hop
      const int sk_grid = static_cast<int>(std::min<long long>(programs, tiles * nkb));
      const double per_prog = std::ceil(static_cast<double>(tiles) * nkb / sk_grid);
      const bool needs_fix = (tiles % sk_grid) != 0;
      double sk = (per_prog * stage_clk + ramp_clk + drain_clk) * clk_to_us;
      if (needs_fix) sk += 2.0 * 128.0 * bn * 4.0 / (hw.fabric_bytes_per_clk * hw.sm_mhz) + hw.flag_us;
      sk = std::max(sk, hbm_floor(static_cast<long long>(sk_grid) * pair)) + hw.launch_us;
      // A wide tile moves a quarter fewer bytes per flop; on long launches the power-limited clock rises by a few percent.
      const double cost = p.streamk ? sk : (halves == 2 ? 0.96 * dp : dp);
      // Prefer, on ties, the wider tile and the pair (fewer fabric bytes per flop).
      if (cost < best_cost * 0.995) {
        best_cost = cost;
        best.bn = bn;
        best.pair = pair;
        best.halves = halves;
        best.dp_us = dp;
        best.sk_us = sk;
        best.grid = static_cast<int>(std::min<long long>(programs, tiles));
        best.sk_grid = sk_grid;
        best.stages = stages;
        const double g = std::sqrt(static_cast<double>(programs) * tile_n / tile_m);
        best.group_m = static_cast<int>(std::max<long long>(1, std::min<long long>(tiles_m, std::llround(g))));
      }
      }  // halves
    }
  }
  if (best_cost >= 1e30) return TB_ERR_UNSUPPORTED;
  std::memset(out, 0, sizeof(*out));
  out->block_m = 128 * best.pair;
  out->block_n = best.bn;
  out->block_k = bk;
  out->group_m = best.group_m;
  out->stages = best.stages;
  out->cta_pair = best.pair;
  out->grid = best.grid;
  out->sk_grid = best.sk_grid;
  out->num_sms = sms;
  out->smem_bytes = smem_bytes_for(best.bn, best.pair, best.stages, best.halves) +
                    (mx ? best.stages * (2 + 2 * 2) * 512 : 0);
  out->tmem_cols = next_pow2(2 * best.bn + (mx ? 8 + 8 * 2 : 0));
  out->predicted_us = static_cast<float>(best.dp_us);
  out->predicted_sk_us = static_cast<float>(best.sk_us);
  out->swap_ab = swap ? 1 : 0;
  out->n_halves = best.halves;
  return TB_OK;
}

}  // namespace tb
