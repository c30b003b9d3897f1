// Machine description and entry point of the analytical selector (see selector.cpp).
#pragma once
#include "../../include/tritonblas_b200.h"

namespace tb {

struct MachineModel {
  int num_sms = 148;             // B200: 2 dies x 74 SMs
  int smem_optin = 232448;       // bytes of shared memory one CTA may opt in to (227 KB)
  double sm_mhz = 1850.0;        // clock the model converts clocks to microseconds with
  double hbm_gbs = 6500.0;       // streaming HBM3e bandwidth
  double fabric_bytes_per_clk = 72.0;  // L2 -> one SM fill rate when few SMs pull
  double l2_bytes_per_clk = 60.0 * 148;  // L2 -> all SMs together (measured: about 60 B/clk per SM with every SM pulling)
  double tile_ramp_clk = 2500.0;       // first TMA round trip + last MMA drain of a program
  double launch_us = 3.0;
  double flag_us = 2.0;          // one global-memory flag hop between programs
  bool allow_pair = true;
};

int select_config(const tb_problem& p, const MachineModel& hw, tb_config* out);
int smem_bytes_for(int block_n, int cta_pair, int stages, int n_halves = 1);

}  // namespace tb
