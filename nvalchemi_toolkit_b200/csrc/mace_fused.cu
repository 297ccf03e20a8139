// SPDX-License-Identifier: Apache-2.0
// Fused MACE convolution for sm_100a: the output layer of the radial MLP runs on the tensor cores INSIDE the
// convolution kernel and its result never leaves the SM.
//
//   R[e, (p, c)] = sum_k h3[e, k] * W4[k, (p, c)]            (tcgen05.mma kind::tf32, accumulator in TMEM)
//   mid[i, :, c] = sum_{e -> i} TP(u[sender(e), :, c], Y(e), R[e, :, c])   (CUDA cores, thread = channel)
//
// One persistent CTA per SM.  The A operand of the MMA is W4^T restricted to a group of at most five paths
// ([paths*128, 64] fp32 = 160 KB, loaded once by TMA and kept resident); the B operand is a tile of FT edges of the
// hidden activations h3 (backward: FT edges x (value, d/dr) = 2 FT rows), streamed by TMA through a two-slot ring.
// D = [128 channels x (paths * rows)] lives in TMEM, double-buffered, so the tensor-core work of tile t+1 overlaps the
// tensor-product arithmetic of tile t.  Thread c of the four compute warps owns TMEM lane c = channel c and reads its
// radial weights with tcgen05.ld (one or two columns per edge and path).  Warp 4 allocates TMEM, issues TMA and MMA.
// Replaces: cuEquivariance fused_tensor_product + the cuBLAS radial MLP output layer of the reference's MACE path
// (nvalchemi/models/mace.py:205-287,403-411), and removes the [E, paths*C] radial-weight round trip through HBM.
// Every mbarrier wait is bounded; on expiry an error code is recorded and the CTA drains and frees its TMEM.
#include "common.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

#include "mace_device.cuh"
#include "mace_tables.h"
#include "tcgen05_utils.cuh"

namespace nva {
using at::Tensor;

constexpr int RECV_BLOCK = 32;  // receivers per work item

template <int LAYER, int GROUP>
struct GroupSpec;
template <>
struct GroupSpec<0, 0> {
  static constexpr int NIN = MACE_L0_NIN, NP = MACE_L0G0_NP, NACC = MACE_L0G0_NACC, NT = MACE_L0G0_NT, NMID = MACE_L0_NMID;
  static __device__ __forceinline__ int mid(int k) { constexpr int m[] = MACE_L0G0_MIDS; return m[k]; }
  static __device__ __forceinline__ void fwd(const float* h, const float* Y, const float* R, float* acc) { MACE_L0G0_FWD(h, Y, R, acc); }
  static constexpr int NZ = MACE_L0G0_NZ;
  static __device__ __forceinline__ void zprep(const float* Y, float* Z) { MACE_L0G0_ZPREP(Y, Z); }
  static __device__ __forceinline__ void fwdz(const float* h, const float* Z, const float* R, float* acc) { MACE_L0G0_FWDZ(h, Z, R, acc); }
  static __device__ __forceinline__ void prep(const float* G, float* T) { MACE_L0G0_BWD_PREP(G, T); }
  static __device__ __forceinline__ void edge(const float* h, const float* Y, const float* R, const float* T, float* dh, float* dY, float* S) { MACE_L0G0_BWD_EDGE(h, Y, R, T, dh, dY, S); }
};
template <>
struct GroupSpec<1, 0> {
  static constexpr int NIN = MACE_L1_NIN, NP = MACE_L1G0_NP, NACC = MACE_L1G0_NACC, NT = MACE_L1G0_NT, NMID = MACE_L1_NMID;
  static __device__ __forceinline__ int mid(int k) { constexpr int m[] = MACE_L1G0_MIDS; return m[k]; }
  static __device__ __forceinline__ void fwd(const float* h, const float* Y, const float* R, float* acc) { MACE_L1G0_FWD(h, Y, R, acc); }
  static constexpr int NZ = MACE_L1G0_NZ;
  static __device__ __forceinline__ void zprep(const float* Y, float* Z) { MACE_L1G0_ZPREP(Y, Z); }
  static __device__ __forceinline__ void fwdz(const float* h, const float* Z, const float* R, float* acc) { MACE_L1G0_FWDZ(h, Z, R, acc); }
  static __device__ __forceinline__ void prep(const float* G, float* T) { MACE_L1G0_BWD_PREP(G, T); }
  static __device__ __forceinline__ void edge(const float* h, const float* Y, const float* R, const float* T, float* dh, float* dY, float* S) { MACE_L1G0_BWD_EDGE(h, Y, R, T, dh, dY, S); }
};
template <>
struct GroupSpec<1, 1> {
  static constexpr int NIN = MACE_L1_NIN, NP = MACE_L1G1_NP, NACC = MACE_L1G1_NACC, NT = MACE_L1G1_NT, NMID = MACE_L1_NMID;
  static __device__ __forceinline__ int mid(int k) { constexpr int m[] = MACE_L1G1_MIDS; return m[k]; }
  static __device__ __forceinline__ void fwd(const float* h, const float* Y, const float* R, float* acc) { MACE_L1G1_FWD(h, Y, R, acc); }
  static constexpr int NZ = MACE_L1G1_NZ;
  static __device__ __forceinline__ void zprep(const float* Y, float* Z) { MACE_L1G1_ZPREP(Y, Z); }
  static __device__ __forceinline__ void fwdz(const float* h, const float* Z, const float* R, float* acc) { MACE_L1G1_FWDZ(h, Z, R, acc); }
  static __device__ __forceinline__ void prep(const float* G, float* T) { MACE_L1G1_BWD_PREP(G, T); }
  static __device__ __forceinline__ void edge(const float* h, const float* Y, const float* R, const float* T, float* dh, float* dY, float* S) { MACE_L1G1_BWD_EDGE(h, Y, R, T, dh, dY, S); }
};

struct FusedArgs {
  int i0, ni;                 // receiver range of this launch
  int64_t e_chunk0;           // first edge covered by the h3 tensor map
  const float* u;
  const float* pos;
  const float* cell;
  const int* batch_idx;
  const int* eptr;
  const int* esend;
  const int* eS;
  float rmax;
  float* mid;                 // forward output
  const float* G;             // backward: dE/dmid
  float* du;                  // backward: feature gradient (may be null)
  float* grad_pos;
  double* virial;
  const int* home_rank;
  const int* home_row;
  const int* row_map;         // optional: sender j reads feature row row_map[j] (rows shared by many atoms, e.g. per species)
  const int64_t* u_ptrs;
  const int64_t* du_ptrs;
  const int64_t* gpos_ptrs;
  int* err;
};

template <int NTHREADS>
__device__ __forceinline__ void compute_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NTHREADS) : "memory"); }

// BWD = false: forward.  BWD = true: adjoint (B rows alternate value / radial derivative, N = 32).
// NG warp-groups of 128 compute threads share one tile: group g takes edges g, g+NG, ... (all groups can read all 128
// TMEM lanes because warp w reaches lanes 32*(w%4)..), keeps its own partial sums and adds them to `mid` with
// reductions.  Four compute warps alone would leave the SM's schedulers with one warp each.
// FT = edges per tile = N of the MMAs (backward: 2 FT).  One tcgen05.mma with M = 128 occupies the tensor pipe for about
// 128 cycles whatever its N (measured: ~175 cycles per instruction at N = 16 and N = 32 alike), so the radial-weight
// GEMM costs paths x 8 x 128 / FT cycles per edge: FT is made as large as the 512 TMEM columns allow with two buffers
// of paths x N columns.
template <int LAYER, int GROUP, bool BWD, bool NEED_DU, int NG, int FT>
__global__ void __launch_bounds__(128 * NG + 64, 1) conv_fused_kernel(const __grid_constant__ CUtensorMap tmW,
                                                            const __grid_constant__ CUtensorMap tmH, FusedArgs a) {
  using G = GroupSpec<LAYER, GROUP>;
  constexpr int NIN = G::NIN, NP = G::NP, NACC = G::NACC, NT = G::NT, NMID = G::NMID;
  constexpr int C = 128;
  constexpr int NROW = BWD ? 2 * FT : FT;            // B rows (= MMA N) per tile
  constexpr uint32_t A_BYTES = NP * 2 * 128 * 128;   // NP paths x 2 k-blocks x [128 rows x 128 B]
  constexpr uint32_t B_BYTES = 2 * NROW * 128;       // 2 k-blocks x [NROW rows x 128 B]
  constexpr uint32_t TCOLS = NP * NROW;              // TMEM columns per buffer
  constexpr uint32_t TALLOC = 2 * TCOLS <= 128 ? 128 : (2 * TCOLS <= 256 ? 256 : 512);
  static_assert(2 * TCOLS <= 512, "TMEM budget");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA = base, sB = base + A_BYTES;
  const uint32_t bar0 = sB + 2 * B_BYTES;
  const uint32_t a_full = bar0, b_full0 = bar0 + 8, b_empty0 = bar0 + 24, t_full0 = bar0 + 40, t_empty0 = bar0 + 56;
  constexpr int GR = FT <= 32 ? 4 : 2;  // depth of the edge-geometry ring (tiles)
  const uint32_t g_full0 = bar0 + 72, g_empty0 = bar0 + 72 + 8 * GR;
  const uint32_t tmem_slot = bar0 + 72 + 16 * GR;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  // per-tile edge data (generic pointers)
  struct __align__(16) TileEdge {
    // backward: M maps dE/dY to the force along the edge (see sh_l3_force_matrix); forward: the same slot holds
    // Z[k] = coef_k * Y[b_k], the channel-independent factor of every coupling term of the path group
    float M[48];
    float Y[16]; float n[3]; float rinv; float v[3]; float f[3];
    int recv; int j; int dup_local; int pad_; const float* up; float* dup; float* gpj;
  };
  static_assert(sizeof(TileEdge) <= 336, "shared-memory budget of the geometry ring");
  static_assert(G::NZ <= 48, "coupling-term factors share the slot of the force matrix");
  TileEdge* te = reinterpret_cast<TileEdge*>(gen + A_BYTES + 2 * B_BYTES + 256);  // [GR][FT]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(reinterpret_cast<uint8_t*>(te) + sizeof(TileEdge) * FT * GR);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int MMA_WARP = 4 * NG, GEO_WARP = 4 * NG + 1;
  const int nwork = (a.ni + RECV_BLOCK - 1) / RECV_BLOCK;

  if (threadIdx.x == 0) {
    mbar_init(a_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(b_full0 + 8 * s, 1); mbar_init(b_empty0 + 8 * s, 1);
      mbar_init(t_full0 + 8 * s, 1); mbar_init(t_empty0 + 8 * s, 4 * NG);
    }
    for (int s = 0; s < GR; ++s) { mbar_init(g_full0 + 8 * s, 1); mbar_init(g_empty0 + 8 * s, 4 * NG); }
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(TALLOC) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ TMA + MMA issuer
    if (lane == 0) {
      mbar_expect_tx(a_full, A_BYTES);
      for (int p = 0; p < NP; ++p)
        for (int kb = 0; kb < 2; ++kb)
          tma_load_2d(sA + (p * 2 + kb) * 128 * 128, &tmW, kb * 32, p * 128, a_full);
      bool ok = mbar_wait(a_full, 0, a.err, 11);
      constexpr uint32_t idesc = umma_idesc_tf32(128, NROW);
      int t = 0;  // global tile counter of this CTA (selects ring slot / TMEM buffer and mbarrier phase)
      // two-deep software pipeline over all tiles of all work items: B(t+1) is requested before MMA(t)
      int w = blockIdx.x, tt = 0, nt_w = 0;
      int64_t row0_w = 0;
      auto open_work = [&](int ww) {
        int i0 = a.i0 + ww * RECV_BLOCK, i1 = min(i0 + RECV_BLOCK, a.i0 + a.ni);
        int e0 = a.eptr[i0], e1 = a.eptr[i1];
        nt_w = (e1 - e0 + FT - 1) / FT;
        row0_w = (int64_t)e0 - a.e_chunk0;
      };
      auto issue_b = [&](int tcount, int64_t erow) -> bool {
        int s = tcount & 1;
        if (!mbar_wait(b_empty0 + 8 * s, ((tcount >> 1) & 1) ^ 1, a.err, 12)) return false;
        mbar_expect_tx(b_full0 + 8 * s, B_BYTES);
        int y = (int)(BWD ? 2 * erow : erow);
        tma_load_2d(sB + s * B_BYTES, &tmH, 0, y, b_full0 + 8 * s);
        tma_load_2d(sB + s * B_BYTES + NROW * 128, &tmH, 32, y, b_full0 + 8 * s);
        return true;
      };
      // iterator over (work item, tile) pairs one step ahead of the MMA
      int pw = w, ptt = 0, pnt = 0;
      int64_t prow0 = 0;
      bool p_valid = false;
      auto advance_prefetch = [&]() {
        // moves (pw, ptt) to the next existing tile; sets p_valid
        while (pw < nwork) {
          if (!p_valid) {
            int i0 = a.i0 + pw * RECV_BLOCK, i1 = min(i0 + RECV_BLOCK, a.i0 + a.ni);
            int e0 = a.eptr[i0], e1 = a.eptr[i1];
            pnt = (e1 - e0 + FT - 1) / FT;
            prow0 = (int64_t)e0 - a.e_chunk0;
            ptt = 0;
            p_valid = true;
          } else {
            ++ptt;
          }
          if (ptt < pnt) return;
          p_valid = false;
          pw += gridDim.x;
        }
      };
      int tp = 0;  // tiles requested so far
      advance_prefetch();
      if (ok && pw < nwork) { ok = issue_b(tp, prow0 + (int64_t)ptt * FT); ++tp; }
      for (; ok && w < nwork; w += gridDim.x) {
        open_work(w);
        for (tt = 0; tt < nt_w && ok; ++tt, ++t) {
          advance_prefetch();
          if (pw < nwork) { ok = issue_b(tp, prow0 + (int64_t)ptt * FT); ++tp; if (!ok) break; }
          int s = t & 1;
          ok = mbar_wait(b_full0 + 8 * s, (t >> 1) & 1, a.err, 13) && mbar_wait(t_empty0 + 8 * s, ((t >> 1) & 1) ^ 1, a.err, 14);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          for (int p = 0; p < NP; ++p) {
            uint32_t d = tmem_base + s * TCOLS + p * NROW;
#pragma unroll
            for (int kb = 0; kb < 2; ++kb)
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                uint64_t da = umma_desc_sw128(sA + (p * 2 + kb) * 128 * 128 + k * UMMA_K * 4);
                uint64_t db = umma_desc_sw128(sB + s * B_BYTES + kb * NROW * 128 + k * UMMA_K * 4);
                umma_tf32(d, da, db, idesc, (kb | k) ? 1u : 0u);
              }
          }
          umma_commit(b_empty0 + 8 * s);
          umma_commit(t_full0 + 8 * s);
        }
      }
      if (!ok) abort_flag[0] = 1;
    }
  } else if (warp == GEO_WARP) {
    // ------------------------------------------------------------------ edge geometry producer (runs GR tiles ahead)
    int t = 0;
    bool ok = true;
    auto flush_forces = [&](int slot) {  // position gradients of a consumed tile: one lane per edge
      if (BWD)
      for (int l = lane; l < FT; l += 32) {
        TileEdge& q = te[slot * FT + l];
        if (q.j >= 0) {
          for (int d = 0; d < 3; ++d) {
            atomicAdd(q.gpj + d, -q.f[d]);
            atomicAdd(a.grad_pos + 3 * (int64_t)q.recv + d, q.f[d]);
          }
          if (a.virial != nullptr) {
            double* vp = a.virial + 9 * (int64_t)a.batch_idx[q.recv];
            for (int x = 0; x < 3; ++x)
              for (int y = 0; y < 3; ++y) atomicAdd(vp + 3 * x + y, (double)(q.v[x] * q.f[y]));
          }
        }
      }
    };
    for (int w = blockIdx.x; w < nwork && ok; w += gridDim.x) {
      int wi0 = a.i0 + w * RECV_BLOCK, wi1 = min(wi0 + RECV_BLOCK, a.i0 + a.ni);
      int e0 = a.eptr[wi0], e1 = a.eptr[wi1];
      int nt_w = (e1 - e0 + FT - 1) / FT;
      int next_recv = wi0;
      for (int tt = 0; tt < nt_w && ok; ++tt, ++t) {
        int gs = t % GR;
        ok = mbar_wait(g_empty0 + 8 * gs, ((t / GR) & 1) ^ 1, a.err, 16);
        if (!ok) break;
        if (t >= GR) flush_forces(gs);
        __syncwarp();
        int tile_e0 = e0 + tt * FT;
        for (int l = lane; l < FT; l += 32) {
          int e = tile_e0 + l;
          TileEdge& q = te[gs * FT + l];
          q.f[0] = 0.f; q.f[1] = 0.f; q.f[2] = 0.f;
          if (e < e1) {
            int i = next_recv;
            while (a.eptr[i + 1] <= e) ++i;  // edges are receiver-major: short forward scan
            int j = a.esend[e];
            float v[3];
            edge_vector(a.pos, a.cell, a.batch_idx, i, j, a.eS + 3 * e, v);
            float r = sqrtf(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]);
            bool in = r < a.rmax && r > 0.f;
            float ri = in ? 1.f / r : 0.f;
            q.n[0] = v[0] * ri; q.n[1] = v[1] * ri; q.n[2] = v[2] * ri; q.rinv = ri;
            q.v[0] = v[0]; q.v[1] = v[1]; q.v[2] = v[2];
            sh_l3(q.n[0], q.n[1], q.n[2], q.Y);
            if (BWD) sh_l3_force_matrix(q.n[0], q.n[1], q.n[2], ri, q.Y, q.M);
            else G::zprep(q.Y, q.M);
            q.recv = i;
            q.j = in ? j : -1;
            const float* ub = a.u;
            float* dub = a.du;
            float* gpb = a.grad_pos;
            int64_t jr = j;
            if (a.home_rank != nullptr) {
              int hr = a.home_rank[j];
              jr = a.home_row[j];
              ub = reinterpret_cast<const float*>(a.u_ptrs[hr]);
              if (BWD && NEED_DU) dub = reinterpret_cast<float*>(a.du_ptrs[hr]);
              if (BWD) gpb = reinterpret_cast<float*>(a.gpos_ptrs[hr]);
            }
            q.up = ub + (a.row_map != nullptr ? (int64_t)a.row_map[j] : jr) * NIN * C;
            q.dup = (BWD && NEED_DU) ? dub + jr * NIN * C : nullptr;
            q.dup_local = dub == a.du ? 1 : 0;
            q.gpj = BWD ? gpb + 3 * jr : nullptr;
          } else {
            q.recv = -1; q.j = -1; q.up = a.u; q.dup = nullptr; q.gpj = nullptr; q.dup_local = 0;
          }
        }
        {
          int last = min(tile_e0 + FT, e1) - 1;
          while (a.eptr[next_recv + 1] <= last) ++next_recv;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(g_full0 + 8 * gs);
      }
    }
    // drain: the last (up to GR) tiles still hold unflushed position gradients
    if (BWD) {
      int first = t > GR ? t - GR : 0;
      for (int tl = first; tl < t; ++tl) {
        if (ok && !mbar_wait(g_empty0 + 8 * (tl % GR), (tl / GR) & 1, a.err, 17)) ok = false;
        if (ok) flush_forces(tl % GR);
      }
    }
    if (!ok && lane == 0) abort_flag[0] = 1;
  } else {
    // ------------------------------------------------------------------ compute warps (thread = channel)
    const int c = threadIdx.x & 127;
    const int grp = warp >> 2, wq = warp & 3;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(wq * 32) << 16);
    int t = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < nwork && ok; w += gridDim.x) {
      int wi0 = a.i0 + w * RECV_BLOCK, wi1 = min(wi0 + RECV_BLOCK, a.i0 + a.ni);
      int e0 = a.eptr[wi0], e1 = a.eptr[wi1];
      int nt_w = (e1 - e0 + FT - 1) / FT;
      int cur = -1;  // receiver whose accumulators are live in this warp-group
      float acc[BWD ? 1 : NACC];
      float T[BWD ? NT : 1];
      for (int tt = 0; tt < nt_w && ok; ++tt, ++t) {
        int s = t & 1, gs = t % GR;
        ok = mbar_wait(g_full0 + 8 * gs, (t / GR) & 1, a.err, 18) && mbar_wait(t_full0 + 8 * s, (t >> 1) & 1, a.err, 15);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        TileEdge* tile = te + gs * FT;
        const uint32_t tb = lane_addr + s * TCOLS;
        // edge loop with the TMEM / global operands of this group's next edge in flight during the current one
        float Rn[BWD ? 2 * NP : NP], hn[NIN];
        auto fetch = [&](int n) {
#pragma unroll
          for (int p = 0; p < NP; ++p) {
            if (BWD) tmem_ld_x2(tb + p * NROW + 2 * n, Rn[p], Rn[NP + p]);
            else tmem_ld_x1(tb + p * NROW + n, Rn[p]);
          }
          const float* up = tile[n].up + c;
#pragma unroll
          for (int k = 0; k < NIN; ++k) hn[k] = __ldg(up + k * C);
        };
        fetch(grp);
        for (int n = grp; n < FT; n += NG) {
          float Rv[NP], Rd[BWD ? NP : 1], h[NIN];
          tmem_ld_wait();
#pragma unroll
          for (int p = 0; p < NP; ++p) { Rv[p] = Rn[p]; if (BWD) Rd[p] = Rn[NP + p]; }
#pragma unroll
          for (int k = 0; k < NIN; ++k) h[k] = hn[k];
          if (n + NG < FT) fetch(n + NG);
          TileEdge& q = tile[n];
          int i = q.recv;
          if (i != cur) {  // uniform across the warp-group
            if (!BWD && cur >= 0) {
              float* mp = a.mid + (int64_t)cur * NMID * C + c;
#pragma unroll
              for (int k = 0; k < NACC; ++k) atomicAdd(mp + G::mid(k) * C, acc[k]);
            }
            cur = i;
            if (i >= 0) {
              if (!BWD) {
#pragma unroll
                for (int k = 0; k < NACC; ++k) acc[k] = 0.f;
              } else {
                float Gr[NACC];
                const float* gp = a.G + (int64_t)i * NMID * C + c;
#pragma unroll
                for (int k = 0; k < NACC; ++k) Gr[k] = gp[G::mid(k) * C];
                G::prep(Gr, T);
              }
            }
          }
          if (!BWD) {
            if (q.j >= 0) G::fwdz(h, q.M, Rv, acc);
          } else if (q.j >= 0) {  // uniform across the warp
            float dh[NIN], dY[16], S[NP], f[3];
#pragma unroll
            for (int k = 0; k < NIN; ++k) dh[k] = 0.f;
#pragma unroll
            for (int b = 0; b < 16; ++b) dY[b] = 0.f;
            G::edge(h, q.Y, Rv, T, dh, dY, S);
            float qq = 0.f;
#pragma unroll
            for (int p = 0; p < NP; ++p) qq = fmaf(S[p], Rd[p], qq);
            // f = qq n + dY . M with the per-edge matrix prepared by the producer warp (48 multiply-adds)
            f[0] = qq * q.n[0]; f[1] = qq * q.n[1]; f[2] = qq * q.n[2];
            const float4* Mp = reinterpret_cast<const float4*>(q.M);
#pragma unroll
            for (int g4 = 0; g4 < 4; ++g4) {  // 4 harmonics = 12 entries = 3 float4 per iteration
              float4 m0 = Mp[3 * g4], m1 = Mp[3 * g4 + 1], m2 = Mp[3 * g4 + 2];
              const float* dy = dY + 4 * g4;
              f[0] = fmaf(dy[0], m0.x, f[0]); f[1] = fmaf(dy[0], m0.y, f[1]); f[2] = fmaf(dy[0], m0.z, f[2]);
              f[0] = fmaf(dy[1], m0.w, f[0]); f[1] = fmaf(dy[1], m1.x, f[1]); f[2] = fmaf(dy[1], m1.y, f[2]);
              f[0] = fmaf(dy[2], m1.z, f[0]); f[1] = fmaf(dy[2], m1.w, f[1]); f[2] = fmaf(dy[2], m2.x, f[2]);
              f[0] = fmaf(dy[3], m2.y, f[0]); f[1] = fmaf(dy[3], m2.z, f[1]); f[2] = fmaf(dy[3], m2.w, f[2]);
            }
            if (NEED_DU) {
              // du is laid out [row][channel][component]: the thread's NIN = 4 gradients are 16 contiguous bytes and go
              // out as ONE vector reduction when the row is in this GPU's memory (a quarter of the L2 atomic
              // operations, which bound this kernel); rows of other GPUs get scalar reductions over NVLink
              float* dp = q.dup + c * NIN;
              if (NIN == 4 && q.dup_local) {
                atomicAdd(reinterpret_cast<float4*>(dp), make_float4(dh[0], dh[NIN > 1 ? 1 : 0], dh[NIN > 2 ? 2 : 0], dh[NIN > 3 ? 3 : 0]));
              } else {
#pragma unroll
                for (int k = 0; k < NIN; ++k) atomicAdd(dp + k, dh[k]);
              }
            }
            {
              // warp sum of the three components with 6 shuffles instead of 15: the first two butterfly stages also
              // split the components over lane groups (lanes 0-7 end up with x, 8-15 with y, 16-23 with z)
              const bool b16 = lane & 16, b8 = lane & 8;
              float k0 = (b16 ? f[2] : f[0]) + __shfl_xor_sync(0xffffffffu, b16 ? f[0] : f[2], 16);
              float k1 = (b16 ? 0.f : f[1]) + __shfl_xor_sync(0xffffffffu, b16 ? f[1] : 0.f, 16);
              float k = (b8 ? k1 : k0) + __shfl_xor_sync(0xffffffffu, b8 ? k0 : k1, 8);
              k += __shfl_xor_sync(0xffffffffu, k, 4);
              k += __shfl_xor_sync(0xffffffffu, k, 2);
              k += __shfl_xor_sync(0xffffffffu, k, 1);
              // shared-memory reduction over the warps of the group: lane 0 holds x, lane 8 y, lane 16 z
              if ((lane & 7) == 0 && lane < 24) atomicAdd(&q.f[lane >> 3], k);
            }
          }
        }
        // every TMEM load of this buffer was waited for: hand the buffer and the geometry slot back
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) { mbar_arrive(t_empty0 + 8 * s); mbar_arrive(g_empty0 + 8 * gs); }
      }
      if (!BWD && cur >= 0 && ok) {
        float* mp = a.mid + (int64_t)cur * NMID * C + c;
#pragma unroll
        for (int k = 0; k < NACC; ++k) atomicAdd(mp + G::mid(k) * C, acc[k]);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TALLOC) : "memory");
  }
}

// ---- host side -------------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 fused_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    C10_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    TORCH_CHECK(p != nullptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is not available");
    fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

static CUtensorMap fused_map(const float* ptr, int64_t rows, int box_rows, int64_t row_stride_floats = 64) {
  CUtensorMap m;
  cuuint64_t dims[2] = {64, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_stride_floats * 4};
  cuuint32_t box[2] = {32, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fused_encode()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", (int)r);
  return m;
}

// tile size: two TMEM buffers of paths x N columns must fit in 512 columns (N = FT forward, 2 FT backward)
template <int LAYER, bool BWD>
struct TileSize { static constexpr int FT = LAYER == 0 ? (BWD ? 32 : 64) : (BWD ? 24 : 48); };

template <int LAYER, int GROUP, bool BWD, bool NEED_DU>
static void launch_fused(const float* wg, int64_t wrows, const float* h3, int64_t hrows, int64_t hstride, const FusedArgs& a, int sms) {
  using G = GroupSpec<LAYER, GROUP>;
  constexpr int FT = TileSize<LAYER, BWD>::FT;
  constexpr int NROW = BWD ? 2 * FT : FT;
  constexpr int GR = FT <= 32 ? 4 : 2;
  static_assert(2 * G::NP * NROW <= 512, "TMEM budget");
  CUtensorMap mw = fused_map(wg, wrows, 128);
  CUtensorMap mh = fused_map(h3, hrows, NROW, hstride);
  size_t smem = (size_t)G::NP * 2 * 128 * 128 + 2 * (2 * NROW * 128) + 256 + GR * FT * 336 + 64 + 1024 + 256;
  constexpr int NG = BWD ? 4 : 5;  // compute warp-groups: both fit their register budgets (96 / 80) without spills; six forward groups measured 0.8 % slower
  auto kern = conv_fused_kernel<LAYER, GROUP, BWD, NEED_DU, NG, FT>;
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  int nwork = (a.ni + RECV_BLOCK - 1) / RECV_BLOCK;
  int grid = std::min(nwork, sms);
  kern<<<grid, 128 * NG + 64, smem, at::cuda::getCurrentCUDAStream()>>>(mw, mh, a);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// wg: [NP*128, 64] = rows of W4^T for the group's paths (path-major); h3: [rows, 64] hidden activations of the chunk's
// edges (backward: value / derivative rows interleaved).  `mid_or_G` is the output (forward) or dE/dmid (backward).
void mace_conv_fused(int64_t layer, int64_t group, bool backward, const Tensor& wg, const Tensor& h3, const Tensor& u,
                     const Tensor& pos, const Tensor& cell, const Tensor& batch_idx, const Tensor& eptr,
                     const Tensor& esend, const Tensor& eS, int64_t i0, int64_t ni, int64_t e_chunk0, double rmax,
                     Tensor mid_or_G, const c10::optional<Tensor>& du, const c10::optional<Tensor>& grad_pos,
                     const c10::optional<Tensor>& virial, const c10::optional<Tensor>& home_rank,
                     const c10::optional<Tensor>& home_row, const c10::optional<Tensor>& u_ptrs,
                     const c10::optional<Tensor>& du_ptrs, const c10::optional<Tensor>& gpos_ptrs, Tensor err,
                     const c10::optional<Tensor>& row_map) {
  c10::cuda::CUDAGuard guard(pos.device());
  NVA_CHECK_CONTIG(wg); NVA_CHECK_CONTIG(u); NVA_CHECK_CONTIG(mid_or_G);
  // h3: contiguous [rows, 64] / [E, 2, 64], or (forward) the value rows of an [E, 2, 64] tensor as a strided [E, 64] view
  TORCH_CHECK(h3.stride(-1) == 1 && (h3.is_contiguous() || (h3.dim() == 2 && !backward && h3.stride(0) % 4 == 0)),
              "mace_conv_fused: h3 must be contiguous or a row-strided 2-D view");
  TORCH_CHECK(u.size(2) == 128, "the fused convolution is specialised for 128 channels");
  TORCH_CHECK(wg.size(1) == 64 && h3.size(-1) == 64, "the fused convolution expects a 64-wide last hidden layer");
  if (ni == 0) return;
  FusedArgs a;
  a.i0 = (int)i0; a.ni = (int)ni; a.e_chunk0 = e_chunk0;
  a.u = u.data_ptr<float>(); a.pos = pos.data_ptr<float>(); a.cell = cell.data_ptr<float>();
  a.batch_idx = batch_idx.data_ptr<int>(); a.eptr = eptr.data_ptr<int>(); a.esend = esend.data_ptr<int>();
  a.eS = eS.data_ptr<int>(); a.rmax = (float)rmax;
  a.mid = backward ? nullptr : mid_or_G.data_ptr<float>();
  a.G = backward ? mid_or_G.data_ptr<float>() : nullptr;
  a.du = du.has_value() ? du->data_ptr<float>() : nullptr;
  a.grad_pos = grad_pos.has_value() ? grad_pos->data_ptr<float>() : nullptr;
  a.virial = virial.has_value() ? virial->data_ptr<double>() : nullptr;
  a.home_rank = home_rank.has_value() ? home_rank->data_ptr<int>() : nullptr;
  a.home_row = home_row.has_value() ? home_row->data_ptr<int>() : nullptr;
  a.row_map = row_map.has_value() ? row_map->data_ptr<int>() : nullptr;
  TORCH_CHECK(!(row_map.has_value() && home_rank.has_value()), "row_map addresses local feature rows only");
  a.u_ptrs = u_ptrs.has_value() ? u_ptrs->data_ptr<int64_t>() : nullptr;
  a.du_ptrs = du_ptrs.has_value() ? du_ptrs->data_ptr<int64_t>() : nullptr;
  a.gpos_ptrs = gpos_ptrs.has_value() ? gpos_ptrs->data_ptr<int64_t>() : nullptr;
  a.err = err.data_ptr<int>();
  const int64_t hrows = h3.numel() / 64, wrows = wg.size(0);
  const int64_t hstride = h3.is_contiguous() ? 64 : h3.stride(0);
  const float *wp = wg.data_ptr<float>(), *hp = h3.data_ptr<float>();
  int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  bool need_du = backward && a.du != nullptr;
#define NVA_CASE(L_, G_)                                                                       \
  if (layer == L_ && group == G_) {                                                            \
    if (!backward) launch_fused<L_, G_, false, false>(wp, wrows, hp, hrows, hstride, a, sms);                         \
    else if (need_du) launch_fused<L_, G_, true, true>(wp, wrows, hp, hrows, hstride, a, sms);                        \
    else launch_fused<L_, G_, true, false>(wp, wrows, hp, hrows, hstride, a, sms);                                    \
    return;                                                                                    \
  }
  NVA_CASE(0, 0)
  NVA_CASE(1, 0)
  NVA_CASE(1, 1)
#undef NVA_CASE
  TORCH_CHECK(false, "mace_conv_fused: unknown (layer, group)");
}

}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("mace_conv_fused(int layer, int group, bool backward, Tensor wg, Tensor h3, Tensor u, Tensor pos, Tensor cell, Tensor batch_idx, Tensor eptr, Tensor esend, Tensor eS, int i0, int ni, int e_chunk0, float rmax, Tensor(a!) mid_or_G, Tensor(b!)? du, Tensor(c!)? grad_pos, Tensor(d!)? virial, Tensor? home_rank, Tensor? home_row, Tensor? u_ptrs, Tensor? du_ptrs, Tensor? gpos_ptrs, Tensor(e!) err, Tensor? row_map=None) -> ()", &nva::mace_conv_fused);
}
