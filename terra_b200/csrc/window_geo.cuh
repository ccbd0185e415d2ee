// Geometry of window attention over the window-major activation layout: where a token of a (possibly shifted)
// window lives (which peer buffer, which row) and which mask region it belongs to. Shared by the attention kernels.
#pragma once
#include "common.cuh"
#include "host_api.h"

namespace tb {

struct Geo {
  int N, nrel;
  int Hg, Wg;  // global token grid
};

// Home of token `tok` of shifted-frame window (ii, jj): which peer slot and which row of its buffer.
struct Home {
  int slot;
  long long row;
  int region;
};

// Debug build: a located token must lie inside the buffer of its slot; otherwise the violation is recorded and the
// location is replaced by row 0 of this rank's own buffer (a valid address), so that the kernel finishes.
__device__ __forceinline__ void check_home(const WindowAttnArgs& a, Home& h, int nwp) {
  if (!TB_DEBUG_BOUNDS) return;
  const int windows = a.tp <= 1 ? nwp : ((nwp + a.tp - 1) / a.tp) * a.tp;
  const long long rows = static_cast<long long>(a.B) * windows * a.shardN;
  const bool ok = h.slot >= 0 && h.slot < a.n_wg * a.sp && h.row >= 0 && h.row < rows;
  if (!tb_index_ok(ok, static_cast<KernelStatus*>(a.debug_status), 0x900u + static_cast<unsigned int>(h.slot & 0xff),
                   static_cast<unsigned int>(h.row), static_cast<unsigned int>(h.row >> 32))) {
    h.slot = a.my_wg * a.sp + a.my_sp;
    h.row = 0;
  }
}

__device__ __forceinline__ Home locate(const WindowAttnArgs& a, const Geo& g, int b, int ii, int jj, int tok) {
  const int ti = tok / a.ww, tj = tok % a.ww;
  const int hs = ii * a.wh + ti, ws = jj * a.ww + tj;  // position in the rolled frame
  int gh = hs + a.sh, gw = ws + a.sw;
  if (gh >= g.Hg) gh -= g.Hg;
  if (gw >= g.Wg) gw -= g.Wg;
  const int flat = (gh / a.wh) * a.nWw + (gw / a.ww);
  const int st = (gh % a.wh) * a.ww + (gw % a.ww);
  int wgr = 0;
  while (wgr + 1 < a.n_wg && flat >= a.win_start[wgr + 1]) ++wgr;
  const int nwp = a.win_start[wgr + 1] - a.win_start[wgr];
  const int lw = flat - a.win_start[wgr];
  const int s = st / a.shardN;
  Home h;
  h.slot = wgr * a.sp + s;
  long long wrow;   // index of (batch, window) among the buffer's windows
  if (a.tp <= 1) {
    wrow = static_cast<long long>(b) * nwp + lw;
  } else {
    // rows gathered over tensor-parallel ranks: chunk t holds [B, wpt windows] of the group, chunks back to back
    const int wpt = (nwp + a.tp - 1) / a.tp;
    const int t = lw / wpt;
    wrow = (static_cast<long long>(t) * a.B + b) * wpt + (lw - t * wpt);
  }
  h.row = wrow * a.shardN + (st - s * a.shardN);
  int rh = 0, rw = 0;
  if (a.sh > 0) rh = hs < g.Hg - a.wh ? 0 : (hs < g.Hg - a.sh ? 1 : 2);
  if (a.sw > 0) rw = ws < g.Wg - a.ww ? 0 : (ws < g.Wg - a.sw ? 1 : 2);
  h.region = rh * 3 + rw;
  check_home(a, h, nwp);
  return h;
}

// The same as `locate` for a token given by its coordinates (ti, tj) inside the window, without the divisions by the
// window size: a shifted token lies in its own window or the next one (per axis), wrapping at the grid end.
__device__ __forceinline__ Home locate_ij(const WindowAttnArgs& a, const Geo& g, int b, int ii, int jj, int ti, int tj) {
  int ri = ti + a.sh, wi = ii;
  if (ri >= a.wh) {
    ri -= a.wh;
    if (++wi == a.nWh) wi = 0;
  }
  int rj = tj + a.sw, wj = jj;
  if (rj >= a.ww) {
    rj -= a.ww;
    if (++wj == a.nWw) wj = 0;
  }
  const int flat = wi * a.nWw + wj;
  const int st = ri * a.ww + rj;
  int wgr = 0;
  while (wgr + 1 < a.n_wg && flat >= a.win_start[wgr + 1]) ++wgr;
  const int nwp = a.win_start[wgr + 1] - a.win_start[wgr];
  const int lw = flat - a.win_start[wgr];
  const int s = a.sp > 1 ? st / a.shardN : 0;
  Home h;
  h.slot = wgr * a.sp + s;
  long long wrow;
  if (a.tp <= 1) {
    wrow = static_cast<long long>(b) * nwp + lw;
  } else {
    const int wpt = (nwp + a.tp - 1) / a.tp;
    const int t = lw / wpt;
    wrow = (static_cast<long long>(t) * a.B + b) * wpt + (lw - t * wpt);
  }
  h.row = wrow * a.shardN + (st - s * a.shardN);
  int rh = 0, rw = 0;
  if (a.sh > 0 && ii == a.nWh - 1) rh = ti < a.wh - a.sh ? 1 : 2;
  if (a.sw > 0 && jj == a.nWw - 1) rw = tj < a.ww - a.sw ? 1 : 2;
  h.region = rh * 3 + rw;
  check_home(a, h, nwp);
  return h;
}

__device__ __forceinline__ int region_of(const WindowAttnArgs& a, const Geo& g, int hs, int ws) {
  int rh = 0, rw = 0;
  if (a.sh > 0) rh = hs < g.Hg - a.wh ? 0 : (hs < g.Hg - a.sh ? 1 : 2);
  if (a.sw > 0) rw = ws < g.Wg - a.ww ? 0 : (ws < g.Wg - a.sw ? 1 : 2);
  return rh * 3 + rw;
}

}  // namespace tb
