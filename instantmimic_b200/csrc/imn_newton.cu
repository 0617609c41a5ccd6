// imn_newton.cu -- the fused Newton constraint solve, one warp per world.
//
// One launch replaces the reference's whole solve pipeline
// (mjw_step_optimized.py:2588-2680): _solve_init_dof, the init of
// newton_fusion.py:431-472 (Jaref, Ma = M qacc, constraint update, gradient,
// Hessian, factor, first search direction), the persistent iteration loop of
// newton_fusion.py:170-296 and the final qfrc_constraint_from_grad.
//
// B200 mapping.  The solve is latency-bound small dense algebra (nv <= 79), not a
// tensor-core contraction, so the design goal is to touch HBM exactly once: a CTA
// is one warp that owns one world.  Its J and row data arrive in shared memory
// through TMA bulk copies (cp.async.bulk, one mbarrier; M, read once per iteration,
// stays in global memory and comes through L1), the Hessian, its
// Cholesky factor and every vector stay on chip for all iterations, and the
// results are written once.  A warp needs no block barrier (only __syncwarp),
// lane reductions are shuffle trees, and the hardware CTA scheduler balances
// worlds whose iteration counts differ; worlds are launched by descending row count
// so that the long solves start first.  Models whose J would leave room for few
// worlds per SM stream it through a 32-row tile (TMA bulk copies from L2) instead.
// The initialisation runs through the same code as an iteration (as "iteration 0"
// without a line search): the kernel is bound by instruction fetch and latency, so
// every stage exists once.
//
// Arithmetic contract.  Every value that decides an active set or an iteration
// count is formed by the same float32 operations in the same order as the CPU
// oracle used by the tests: explicit fmaf chains in ascending index order,
// shuffle-down trees for lane sums, IEEE sqrt and division.  Blocking, register
// tiling and the lane mapping never change the order in which one value
// receives its terms.
#include <stdio.h>

#include "imn_newton_factor.cuh"
#include "imn_newton_ls.cuh"

namespace imn {

// Phase timers, compiled only into the profiling build (-DIMN_PROFILE).
#ifdef IMN_PROFILE
__device__ unsigned long long g_prof[16];
#define PROF_DECL long long prof_t = clock64(); long long prof_acc[16] = {0}; s.prof_acc = prof_acc; s.prof_t = &prof_t
#define PROF(k) do { const long long t_ = clock64(); prof_acc[k] += t_ - prof_t; prof_t = t_; } while (0)
#define PROF_FLUSH do { if (lane == 0) for (int k_ = 0; k_ < 16; ++k_) atomicAdd(&g_prof[k_], (unsigned long long)prof_acc[k_]); } while (0)
#else
#define PROF_DECL
#define PROF(k)
#define PROF_FLUSH
#endif

// Internal error bit OR-ed into `overflow` when the input copies of a world do not
// complete within the wait limit (the world is left unsolved).
#define IMN_OVERFLOW_COPY_TIMEOUT (1 << 30)

struct Geom {
  int nv, njmax, ldj, ldu, nM, bd;
  int jrows;  // rows of J held in shared memory (njmax when resident, else 32)
  // offsets in 4-byte words; every region starts on a 16-byte boundary
  int oBar, oJ, oA, oVec, nv4, oRowF, oRowI, r4, oUni, total;
  // polls a copy wait may take before the world gives up, and the failure-path test
  // switch: when set no bulk copy is issued (plain loads bring the data) while the
  // barrier is told to expect bytes, so the wait runs out with nothing in flight
  int wait_polls, withhold_copies;
};

// Set by imn_set_copy_wait_limit; read when a launch is planned.
static int g_wait_polls = 1 << 22;
static int g_withhold_copies = 0;


static inline int up4(int n) { return (n + 3) & ~3; }

static Geom make_geom(const ImnModel& m, const ImnData& d, bool resident, const ImnSparsePlan* sp = nullptr) {
  Geom g;
  g.nv = m.nv;
  g.njmax = d.njmax;
  g.ldj = (int)d.J_ld_row;
  g.ldu = up4(m.nv + 1);
  g.nM = m.nM;
  g.bd = m.nv_pad >= 64 ? 64 : 32;
  g.jrows = resident ? d.njmax : 32;
  g.nv4 = up4(m.nv);
  g.r4 = up4(d.njmax);
  int o = 0;
  g.oBar = o, o += 4;
  // a streamed tile may start up to three floats into its buffer and end on a 16-byte boundary
  g.oJ = o, o += up4(g.jrows * g.ldj) + (resident ? 0 : 8);
  // dense: H and its factor share one (nv+1) x ldu array; sparse plan: packed H | N | 1/D
  g.oA = o, o += sp ? up4(sp->nfac) + up4(sp->nslots) + up4(m.nv) : (m.nv + 1) * g.ldu;
  // dof vectors; the dense factor needs two more (forward-solve scratch, 1 / pivot)
  g.oVec = o, o += (sp ? 6 : 8) * g.nv4;
  g.oRowF = o, o += 5 * g.r4;
  g.oRowI = o, o += up4(3 * g.r4 / 2);  // three 16-bit row lists
  g.oUni = o, o += up4(m.nv + 1);
  g.total = o;
  g.wait_polls = g_wait_polls;
  g.withhold_copies = g_withhold_copies;
  return g;
}

// The two overflow warnings of the reference (newton_stages.py:430-436, newton_fusion.py:283-289),
// kept out of line (measured 0.6 % faster than inline).
__device__ __noinline__ void warn_limit(int which, unsigned limit) {
  if (which == 0)
    printf("linesearch iterations limit reached - please increase ls_iterations to %u\n", limit);
  else
    printf("solver iterations limit reached - please increase iterations to %u\n", limit);
}

// One warp solves one world: the CTA's.  The solve is written as one loop whose trip is
// "take the world if none is in hand, else run one pass of it" rather than as a load
// followed by a pass loop: the same statements, but the compiler lays the single loop
// out better (measured: 0.836 -> 0.796 ms per 8192 humanoid worlds at the same
// occupancy).
template <bool JRES, bool SPARSE, bool STATS>
__device__ __forceinline__ void newton_worlds(const ImnModel& m, const ImnData& d, const ImnCtx& cx, const Geom& g,
                                              const ImnSparsePlan& sp) {
  extern __shared__ __align__(16) float smem[];
  const int lane = threadIdx.x;
  const int nv = g.nv, R = g.njmax, nv4 = g.nv4, r4 = g.r4;

  void* bar = smem + g.oBar;
  World s;
  s.nv = nv, s.ldj = g.ldj, s.ldu = g.ldu, s.bd = g.bd, s.lane = lane, s.nM = g.nM;
  s.Jsm = smem + g.oJ;
  s.A = smem + g.oA;
  s.qacc = smem + g.oVec;
  s.Ma = s.qacc + nv4;
  s.search = s.Ma + nv4;
  s.mv = s.search + nv4;
  s.grad = s.mv + nv4;
  s.qfs = s.grad + nv4;
  s.xsm = SPARSE ? nullptr : s.qfs + nv4;
  s.dinv = SPARSE ? nullptr : s.xsm + nv4;
  s.Jaref = smem + g.oRowF;
  s.jv = s.Jaref + r4;
  s.Dsm = s.jv + r4;
  s.floss = s.Dsm + r4;
  s.force = s.floss + r4;
  s.state = reinterpret_cast<uint16_t*>(smem + g.oRowI);
  s.ids = s.state + r4;
  s.frows = s.ids + r4;  // rows with a nonzero force, ascending
  s.uni = reinterpret_cast<int*>(smem + g.oUni);
  s.mulm_rowadr = m.M_mulm_rowadr;
  s.mulm_pack = m.M_mulm_pack;
  s.jbar = bar;
  s.jphase = reinterpret_cast<int*>(smem + g.oBar) + 2;  // the barrier itself takes two words
  s.jfail = s.jphase + 1;
  s.wait_polls = g.wait_polls, s.withhold_copies = g.withhold_copies;
  s.Hp = s.A;
  s.N = s.A + (SPARSE ? ((sp.nfac + 3) & ~3) : 0);
  s.iD = s.N + (SPARSE ? ((sp.nslots + 3) & ~3) : 0);
  s.Jbeg = d.efc_J;
  s.Jend = d.efc_J + (d.J_world_offset ? (size_t)d.J_elems
                                       : (size_t)(d.nworld - 1) * d.J_ld_world + (size_t)d.njmax * d.J_ld_row);
  if (lane == 0) mbar_init(bar, 1);
  __syncwarp();

  PROF_DECL;
  // the world in hand
  int w = 0, nefc = 0, ne = 0, nef = 0;
  bool rowless = false;
  size_t dofo = 0, efco = 0;
  float tolerance = 0.0f, ls_tolerance = 0.0f, scale = 1.0f;
  float search_dot = 0.0f, grad_dot = 0.0f, grad_scale = 1.0f, decrement = 0.0f;
  float improvement = 0.0f, alpha = 0.0f;
  int quad_count = 0, state_count = 0, niter = 0, overflow = 0;
  bool search_unchanged = false, ls_exhausted = false;
  int st_passes = 0, st_flips = 0, st_factor = 0, st_grad = 0;  // work counters (ctx.stats)
  bool have = false, first = true;
  bool taken = false;  // this CTA's world was taken

#pragma unroll 1
  for (;;) {
    if (!have && !taken) {
      // ---- take the world ------------------------------------------------------------
      taken = true;
      {
        const int idx = (int)blockIdx.x;
        w = cx.world_order ? cx.world_order[idx] : idx;
        s.world = w;
        s.viol = (SPARSE && cx.hfactor) ? cx.hfactor + ((size_t)w + 1) * m.nv_pad * m.nv_pad - 1 : nullptr;
        const int nefc_in = d.nefc[w];
        nefc = min(R, nefc_in);
        ne = d.ne[w], nef = ne + d.nf[w];
        s.nefc = nefc, s.ne = ne, s.nef = nef;
        rowless = nefc_in == 0;
        dofo = (size_t)w * d.dof_ld, efco = (size_t)w * d.efc_ld;
        s.Jg = d.efc_J + (d.J_world_offset ? (size_t)d.J_world_offset[w] : (size_t)w * d.J_ld_world);
        s.M = d.M + (size_t)w * d.M_ld;

        // ---- load: TMA bulk copies for the 16-byte-aligned bulk of every array, plain
        // loads for the ragged ends ---------------------------------------------------
        const float* q0 = (m.warmstart && !rowless) ? d.qacc_warmstart : d.qacc_smooth;
        struct Src {
          float* dst;
          const float* src;
          int n;
        };
        const Src srcs[6] = {
            {s.Jsm, s.Jg, JRES ? nefc * s.ldj : 0},
            {s.Dsm, d.efc_D + efco, nefc},
            {s.floss, d.efc_frictionloss + efco, nefc},
            {s.jv, d.efc_aref + efco, nefc},  // aref is parked in jv until Jaref is formed
            {s.qacc, q0 + dofo, nv},
            {s.qfs, d.qfrc_smooth + dofo, nv},
        };
        if (lane == 0) {
          *s.jphase = 1;  // phase 0 is the load below
          *s.jfail = 0;
        }
        __syncwarp();
        const bool bulk = !(g.withhold_copies & 1);
        uint32_t tx = 0;
#pragma unroll
        for (int k = 0; k < 6; ++k)
          if (bulk && (reinterpret_cast<uintptr_t>(srcs[k].src) & 15) == 0) tx += (uint32_t)(srcs[k].n & ~3) * 4u;
        if (lane == 0) {
          mbar_expect_tx(bar, bulk ? tx : 16u);
#pragma unroll
          for (int k = 0; k < 6; ++k) {
            const uint32_t bytes =
                bulk && (reinterpret_cast<uintptr_t>(srcs[k].src) & 15) == 0 ? (uint32_t)(srcs[k].n & ~3) * 4u : 0u;
            if (bytes) bulk_g2s(srcs[k].dst, srcs[k].src, bytes, bar);
          }
        }
#pragma unroll
        for (int k = 0; k < 6; ++k) {
          const int done_n = bulk && (reinterpret_cast<uintptr_t>(srcs[k].src) & 15) == 0 ? (srcs[k].n & ~3) : 0;
#pragma unroll 1
          for (int i = done_n + lane; i < srcs[k].n; i += 32) srcs[k].dst[i] = srcs[k].src[i];
        }
#pragma unroll 1
        for (int i = lane; i < nv; i += 32) s.search[i] = 0.0f, s.mv[i] = 0.0f, s.grad[i] = 0.0f;
#pragma unroll 1
        for (int i = lane; i <= nv; i += 32) s.uni[i] = 0;
        // bounded wait for the copies; when it runs out the copies get one more bounded wait
        // (they write this CTA's shared memory, which the SM hands to the next CTA once
        // this one is gone), then the world is left unsolved with the time-out bit set
        bool arrived = false;
#pragma unroll 1
        for (int tries = 0; tries < g.wait_polls && !arrived; ++tries) arrived = mbar_try_wait(bar, 0);
        if (!arrived) {
#pragma unroll 1
          for (int tries = 0; tries < g.wait_polls && !arrived; ++tries) arrived = mbar_try_wait(bar, 0);
          if (lane == 0) d.overflow[w] |= IMN_OVERFLOW_COPY_TIMEOUT;
        } else {
          have = true, first = true;
          search_dot = 0.0f, grad_dot = 0.0f, grad_scale = 1.0f, decrement = 0.0f;
          improvement = 0.0f, alpha = 0.0f;
          quad_count = 0, state_count = 0, niter = 0, overflow = 0;
          search_unchanged = false, ls_exhausted = false;
          if (STATS) st_passes = 0, st_flips = 0, st_factor = 0, st_grad = 0;
          tolerance = m.opt_tolerance[w % m.n_tolerance];
          ls_tolerance = m.opt_ls_tolerance[w % m.n_ls_tolerance];
          scale = m.stat_meaninertia[w % m.n_meaninertia] * (float)nv;
        }
        __syncwarp();
        PROF(0);
      }
    }
    if (!have) break;

    // Pass 0 is the initialisation (newton_fusion.py:431-472): Jaref = J qacc - aref,
    // Ma = M qacc, row states, gradient, full Hessian, factor, first search direction.
    // Every later pass is one Newton iteration (newton_fusion.py:170-296).
    bool finished = false, failed = false;
    do {
      // one call site: Ma = M qacc, Jaref = J qacc - aref on pass 0; mv = M search,
      // jv = J search afterwards
      if (first || !search_unchanged)
        products<JRES>(s, first ? s.qacc : s.search, first ? s.Ma : s.mv, first ? s.Jaref : s.jv,
                       first ? s.jv : nullptr);
      __syncwarp();
      PROF(5);
      if (rowless) {
        finished = true;
        break;
      }
      float noise_floor = 0.0f;
      bool ls_converged = true;
      if (!first) {
        const LineSearchResult ls =
            line_search(s, search_dot, tolerance, ls_tolerance, scale, m.alpha_noise_eps, m.ls_iterations);
        alpha = ls.alpha, improvement = ls.improvement, noise_floor = ls.noise_floor;
        ls_converged = ls.converged;
        if (STATS) st_passes += ls.passes;
#pragma unroll 1
        for (int i = lane; i < nv; i += 32) {
          s.qacc[i] = fmaf(alpha, s.search[i], s.qacc[i]);
          s.Ma[i] = fmaf(alpha, s.mv[i], s.Ma[i]);
        }
      }
      PROF(6);
      // ---- move along the search direction, re-evaluate rows, list QUADRATIC flips
      // (newton_stages.py:373-426); on pass 0 this is upstream's constraint update
      quad_count = 0;
      state_count = 0;
      int nfr = 0;
#pragma unroll 1
      for (int base = 0; base < nefc; base += 32) {
        const int r = base + lane;
        bool flip = false, changed = false;
        float f = 0.0f;
        if (r < nefc) {
          const float nj = first ? s.Jaref[r] : rounded_step(s.Jaref[r], alpha, s.jv[r]);
          s.Jaref[r] = nj;
          const bool is_eq = r < ne, is_fr = !is_eq && r < nef;
          int ns;
          eval_constraint(is_eq, is_fr, nj, s.Dsm[r], is_fr ? s.floss[r] : 0.0f, f, ns);
          const int old = first ? -1 : s.state[r];
          s.force[r] = f;
          s.state[r] = ns;
          if (first) s.jv[r] = 0.0f;  // aref no longer needed
          // pass 0 lists every QUADRATIC row (the rows of the full Hessian, whatever their
          // force: a row at Jaref == 0 has no force but still carries D J^T J); later
          // passes list the rows whose QUADRATIC membership flipped
          flip = first ? ns == IMN_STATE_QUADRATIC
                       : (old == IMN_STATE_QUADRATIC) != (ns == IMN_STATE_QUADRATIC);
          changed = old != ns;
        }
        const unsigned below = (1u << lane) - 1u;
        const unsigned fm = __ballot_sync(IMN_FULL_MASK, flip);
        if (flip) s.ids[quad_count + __popc(fm & below)] = r;
        quad_count += __popc(fm);
        state_count += __popc(__ballot_sync(IMN_FULL_MASK, changed));
        const unsigned nz = __ballot_sync(IMN_FULL_MASK, f != 0.0f);
        if (f != 0.0f) s.frows[nfr + __popc(nz & below)] = r;
        nfr += __popc(nz);
      }
      if (!first) {
        ls_exhausted = fabsf(alpha) < noise_floor;
        if (ls_exhausted) state_count += 1;
        if (!ls_converged) {
          if ((m.warn_overflow & m.overflow_ls_iterations) && lane == 0) warn_limit(0, (unsigned)m.ls_iterations);
          overflow |= m.overflow_ls_iterations;
        }
      }
      __syncwarp();
      PROF(7);
      // ---- gradient (newton_stages.py:745-798), Hessian, factor (newton_stages.py:629-740)
      const bool changed = first || state_count != 0;
      search_unchanged = !changed;
      if (!changed) {
        const float sigma = grad_scale, ns = sigma - alpha;
        const float ratio = sigma != 0.0f ? ns / sigma : 0.0f;
        const float rsq = ratio * ratio;
        grad_dot *= rsq;
        decrement *= rsq;
        grad_scale = ns;
      } else {
        grad_dot = full_gradient<JRES>(s, nfr);
        if (STATS) {
          ++st_grad;
          if (!first) st_flips += quad_count;
          if (first || quad_count > 0) ++st_factor;
        }
        PROF(8);
        decrement = 0.0f;
        grad_scale = 1.0f;
        if (first) {
          if (SPARSE)
            assemble_hessian_sparse<JRES>(s, quad_count, sp);
          else
            assemble_hessian<JRES>(s, quad_count);
        } else if (quad_count > 0) {
          update_hessian<JRES, SPARSE>(s, quad_count, sp);
        }
        PROF(9);
        if (SPARSE) {
          // refactor the packed H, or solve with the resident factor
          // (sparse_hessian.py:490-547)
          if (first || quad_count > 0) {
            if (!first) {
#pragma unroll 1
              for (int q = lane; q < sp.nfac; q += 32) s.N[q] = s.Hp[q];
            }
            sp_load_rhs(sp, s.N, s.grad, lane);
            IMN_MARK(s, 1);
            sp_factor_sweeps(sp, s.N, s.iD, lane);
            IMN_MARK(s, 2);
          } else {
            sp_forward(sp, s.N, s.iD, s.grad, lane);
            IMN_MARK(s, 3);
          }
          sp_backward_sweeps(sp, s.N, s.iD, s.grad, s.search, s.bd, lane, search_dot, decrement);
          IMN_MARK(s, 4);
        } else {
          factor_solve(s, first || quad_count > 0, search_dot, decrement);
        }
        PROF(10);
      }
      if (!JRES && *s.jfail) {
        // a tile copy of this pass did not complete within its wait limit, so the pass
        // worked on stale rows: give the copy one more bounded wait (it writes this
        // CTA's shared memory), then leave the world unsolved, results unwritten
        const uint32_t parity = (uint32_t)*s.jphase ^ 1u;
        bool arrived = false;
#pragma unroll 1
        for (int tries = 0; tries < g.wait_polls && !arrived; ++tries) arrived = mbar_try_wait(bar, parity);
        if (lane == 0) d.overflow[w] |= IMN_OVERFLOW_COPY_TIMEOUT;
        finished = true, failed = true;
        break;
      }
      if (first) {
        quad_count = 0, state_count = 0;
        break;
      }
      // ---- convergence (newton_fusion.py:267-295) -------------------------------
      ++niter;
      const bool converged = alpha == 0.0f || (improvement > 0.0f && improvement / scale < tolerance) ||
                             sqrtf(grad_dot) / scale < tolerance ||
                             0.5f * decrement / scale < tolerance;
      if (converged || niter == m.iterations) {
        if (!converged) {
          if ((m.warn_overflow & m.overflow_iterations) && lane == 0) warn_limit(1, (unsigned)m.iterations);
          overflow |= m.overflow_iterations;
        }
        if (lane == 0 && cx.nsolving) atomicAdd(cx.nsolving, -1);
        finished = true;
      }
    } while (false);
    first = false;
    if (!finished) continue;
    have = false;
    if (failed) continue;

    // ---- results (once) ---------------------------------------------------------
#pragma unroll 1
    for (int i = lane; i < nv; i += 32) {
      d.qacc[dofo + i] = s.qacc[i];
      d.efc_Ma[dofo + i] = s.Ma[i];
      d.qfrc_constraint[dofo + i] = rowless ? 0.0f : fmaf(-grad_scale, s.grad[i], s.Ma[i] - s.qfs[i]);
      if (cx.search) cx.search[dofo + i] = s.search[i];
      if (cx.mv) cx.mv[dofo + i] = s.mv[i];
      if (cx.grad) cx.grad[(size_t)w * cx.grad_ld + i] = s.grad[i];
    }
#pragma unroll 1
    for (int r = lane; r < nefc; r += 32) {
      d.efc_force[efco + r] = s.force[r];
      d.efc_state[efco + r] = s.state[r];
      if (cx.Jaref) cx.Jaref[efco + r] = s.Jaref[r];
      if (cx.jv) cx.jv[efco + r] = s.jv[r];
      if (cx.quad_changed_ids && r < quad_count) cx.quad_changed_ids[efco + r] = s.ids[r];
    }
    if (cx.dof_union && !rowless)
#pragma unroll 1
      for (int i = lane; i <= nv; i += 32) cx.dof_union[(size_t)w * (nv + 1) + i] = s.uni[i];
    if (SPARSE && !rowless && cx.hfactor && cx.h) {
      // packed H | N | 1/D, the reference's hfactor layout (sparse_hessian.py:488-489).
      // The factor never leaves the chip here, so it is written only for callers that
      // inspect the context (those that also pass ctx.h); the violation counter in the
      // last element is always live.
      float* Uf = cx.hfactor + (size_t)w * m.nv_pad * m.nv_pad;
#pragma unroll 1
      for (int q = lane; q < sp.nfac; q += 32) Uf[q] = s.Hp[q], Uf[sp.nfac + q] = s.N[q];
#pragma unroll 1
      for (int q = lane; q < nv; q += 32) Uf[2 * sp.nfac + q] = s.iD[q];
    }
    if (!SPARSE && !rowless) {
      const size_t ho = (size_t)w * m.nv_pad * m.nv_pad;
      if (cx.h)
#pragma unroll 1
        for (int r = 0; r < nv; ++r)
#pragma unroll 1
          for (int c = r + lane; c < nv; c += 32) cx.h[ho + (size_t)r * m.nv_pad + c] = s.A[(c + 1) * s.ldu + r];
      if (cx.hfactor)
#pragma unroll 1
        for (int r = 0; r < nv; ++r)
#pragma unroll 1
          for (int c = r + lane; c < nv; c += 32) cx.hfactor[ho + (size_t)r * m.nv_pad + c] = s.A[r * s.ldu + c];
    }
    PROF(11);
    if (lane == 0) {
      d.solver_niter[w] = niter;
      if (overflow) d.overflow[w] |= overflow;
      if (cx.search_dot) cx.search_dot[w] = search_dot;
      if (cx.done) cx.done[w] = 1;
      if (STATS && cx.stats) {
        int4 st = make_int4(st_passes, st_flips, st_factor, st_grad);
        *reinterpret_cast<int4*>(cx.stats + 4 * (size_t)w) = st;
      }
      if (!rowless) {
        if (cx.grad_dot) cx.grad_dot[w] = grad_dot;
        if (cx.grad_scale) cx.grad_scale[w] = grad_scale;
        if (cx.newton_decrement) cx.newton_decrement[w] = decrement;
        if (cx.improvement) cx.improvement[w] = improvement;
        if (cx.alpha) cx.alpha[w] = alpha;
        if (cx.search_unchanged) cx.search_unchanged[w] = search_unchanged;
        if (cx.ls_exhausted) cx.ls_exhausted[w] = ls_exhausted;
        if (cx.quad_changed_count) cx.quad_changed_count[w] = quad_count;
        if (cx.state_changed_count) cx.state_changed_count[w] = state_count;
      }
    }
    __syncwarp();
  }
  PROF_FLUSH;
}

// Two entry points over the same body.  With J resident shared memory limits the worlds
// per SM to about 14 at the humanoid's shapes; the register bound is set to match
// (14 one-warp CTAs per SM: 144 registers, no spills).  Measured per 8192 humanoid worlds
// with this bound at 1 (148 registers, one warp fewer per SM) 0.902 ms, 12: 0.899,
// 13: 0.795, 14: 0.797, 15: 0.800, 16: 0.803.  The streamed variants hold more worlds per
// SM in shared memory than an uncapped register count would allow, so theirs is capped at
// 128 (16 warps per SM).
// STATS compiles the work counters of ImnCtx.stats in: four more live values in a
// kernel that is short of registers cost 9 % of its speed (measured), so the counting
// variants run only for callers that pass the stats array.
#ifndef IMN_RESIDENT_MIN_BLOCKS
#define IMN_RESIDENT_MIN_BLOCKS 14
#endif
template <bool SPARSE, bool STATS>
__global__ void __launch_bounds__(32, IMN_RESIDENT_MIN_BLOCKS) newton_kernel_resident(const ImnModel m, const ImnData d, const ImnCtx cx,
                                                                   const Geom g, const ImnSparsePlan sp) {
  newton_worlds<true, SPARSE, STATS>(m, d, cx, g, sp);
}
#ifndef IMN_STREAMED_MIN_BLOCKS
#define IMN_STREAMED_MIN_BLOCKS 12
#endif
template <bool SPARSE, bool STATS>
__global__ void __launch_bounds__(32, IMN_STREAMED_MIN_BLOCKS) newton_kernel_streamed(const ImnModel m, const ImnData d, const ImnCtx cx,
                                                                 const Geom g, const ImnSparsePlan sp) {
  newton_worlds<false, SPARSE, STATS>(m, d, cx, g, sp);
}

__global__ void fill_nsolving(int* nsolving, int value) { *nsolving = value; }

// The hardware hands CTAs to SMs in index order and a world's solve time grows with
// its row count, so worlds are launched by descending row count: the long solves
// start first and the launch ends with short ones instead of a few stragglers.  One
// CTA sorts the worlds into 64 classes of row count (counting sort through shared
// memory); the order inside a class depends on atomics and is irrelevant: every
// world is solved independently of which CTA takes it.
#define IMN_ORDER_CLASSES 64
__global__ void __launch_bounds__(1024) order_worlds_kernel(const int* __restrict__ nefc, int njmax, int nworld,
                                                            int* __restrict__ order, int* nsolving) {
  __shared__ int count[IMN_ORDER_CLASSES], start[IMN_ORDER_CLASSES];
  const int tid = threadIdx.x;
  if (tid < IMN_ORDER_CLASSES) count[tid] = 0;
  if (tid == 0 && nsolving) *nsolving = nworld;
  __syncthreads();
  // class 0 holds the largest row counts
  auto cls = [&](int n) {
    n = min(max(n, 0), njmax);
    return (int)(((long long)(njmax - n) * IMN_ORDER_CLASSES) / (njmax + 1));
  };
  for (int w = tid; w < nworld; w += blockDim.x) atomicAdd(&count[cls(nefc[w])], 1);
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int c = 0; c < IMN_ORDER_CLASSES; ++c) start[c] = run, run += count[c];
  }
  __syncthreads();
  for (int w = tid; w < nworld; w += blockDim.x) order[atomicAdd(&start[cls(nefc[w])], 1)] = w;
}

// Largest dynamic shared memory one CTA may opt into on sm_100 (227 KB).
static const int kMaxSmem = 227 * 1024;
// Resident-J budget per world: keep at least 4 worlds per SM.
static const int kResidentBudget = kMaxSmem / 4;

static int validate(const ImnModel* m, const ImnData* d, const ImnCtx* cx) {
  if (!m || !d || !cx) return set_error("imn_solve: NULL struct"), IMN_ERR_NULL;
  if (d->nworld < 0 || d->njmax < 0) return set_error("imn_solve: negative extent"), IMN_ERR_SHAPE;
  if (d->njmax >= (1 << 16)) return set_error("imn_solve: njmax %d exceeds 16-bit row indices", d->njmax), IMN_ERR_LIMIT;
  if (m->nv <= 0 || m->nv > 79 || m->nv_pad % 16 != 0 || m->nv_pad > 80 || m->nv_pad <= m->nv)
    return set_error("imn_solve: nv %d / nv_pad %d outside the fused path (0 < nv <= 79, nv_pad %% 16 == 0, nv < nv_pad <= 80)",
                     m->nv, m->nv_pad),
           IMN_ERR_UNSUPPORTED;
  if (m->iterations <= 0) return set_error("imn_solve: iterations must be positive"), IMN_ERR_UNSUPPORTED;
  if (m->n_tolerance <= 0 || m->n_ls_tolerance <= 0 || m->n_meaninertia <= 0)
    return set_error("imn_solve: empty option array"), IMN_ERR_SHAPE;
  const void* need[] = {m->opt_tolerance, m->opt_ls_tolerance, m->stat_meaninertia, m->M_mulm_rowadr,
                        m->M_mulm_pack, d->nefc, d->ne, d->nf, d->qacc_smooth, d->qacc_warmstart,
                        d->qfrc_smooth, d->efc_J, d->efc_D, d->efc_aref, d->efc_frictionloss, d->M, d->qacc,
                        d->qfrc_constraint, d->efc_Ma, d->efc_force, d->efc_state, d->solver_niter,
                        d->overflow};
  for (const void* p : need)
    if (!p) return set_error("imn_solve: a required Model/Data pointer is NULL"), IMN_ERR_NULL;
  if (d->dof_ld < m->nv || d->J_ld_row < m->nv || d->efc_ld < d->njmax || d->M_ld < m->nM ||
      (!d->J_world_offset && d->J_ld_world < (int64_t)d->njmax * d->J_ld_row) ||
      (d->J_world_offset && d->J_elems < 0))
    return set_error("imn_solve: a stride is smaller than its extent"), IMN_ERR_SHAPE;
  if (d->J_ld_row > 4 * (int64_t)m->nv + 64)
    return set_error("imn_solve: efc.J row stride %lld is far larger than nv %d", (long long)d->J_ld_row, m->nv),
           IMN_ERR_SHAPE;
  if (m->nM >= (1 << 16)) return set_error("imn_solve: nM exceeds 16-bit indices"), IMN_ERR_LIMIT;
  if (cx->grad && cx->grad_ld < m->nv) return set_error("imn_solve: ctx.grad stride < nv"), IMN_ERR_SHAPE;
  if (cx->sparse_plan) {
    const ImnSparsePlan* sp = cx->sparse_plan;
    if (sp->nv != m->nv || sp->nv_pad != m->nv_pad || sp->nfac <= 0 || sp->nslots != sp->nfac + sp->nv ||
        2 * sp->nfac + sp->nv >= sp->nv_pad * sp->nv_pad - 1 || sp->nlevels <= 0)
      return set_error("imn_solve: sparse plan does not match the model"), IMN_ERR_SHAPE;
    if (!cx->hfactor) return set_error("imn_solve: the sparse path needs ctx.hfactor (violation counter)"), IMN_ERR_NULL;
    if (!sp->lvl_ptr || !sp->lvl_team || !sp->ent_slot || !sp->ent_col || !sp->run_ptr || !sp->run_ab ||
        !sp->run_kl || !sp->orig || !sp->b_lvl || !sp->b_slot || !sp->b_src || !sp->b_dst || !sp->pair ||
        !sp->f_lvl || !sp->f_row || !sp->row_start || !sp->rk_ptr || !sp->rk || !sp->pmask || !sp->s_a ||
        !sp->s_b || !sp->s_m || !sp->fsweep || !sp->bsweep || sp->nfsweep <= 0 || sp->nbsweep < 0)
      return set_error("imn_solve: a sparse plan table is NULL"), IMN_ERR_NULL;
  }
  return IMN_OK;
}

// Worlds one SM holds at `bytes` of dynamic shared memory per one-warp CTA (1 KB is
// reserved per CTA; `cap` is the register limit of the kernel variant).
static int worlds_per_sm(int bytes, int cap = 16) {
  const int n = (228 * 1024) / (bytes + 1024);
  return n < cap ? n : cap;
}

// J resident in shared memory or streamed through the 32-row tile.  Resident J is
// read once from HBM; a streamed J is re-read from L2 in every stage but leaves room
// for more worlds per SM.  Measured on B200 (dense factor): humanoid (njmax 64) 12
// resident vs 16 streamed worlds per SM: resident 7 % faster; SNU-like (njmax 128) 4 vs
// 7: streamed 1.22x faster; G1-like (njmax 250) 4 vs 11: streamed 1.6x faster.  Hence:
// stream when it holds at least 1.6x the worlds.
static int plan_launch(const ImnModel* m, const ImnData* d, const ImnSparsePlan* sp, Geom* g, bool* resident) {
  const Geom gr = make_geom(*m, *d, true, sp);
  const Geom gs = make_geom(*m, *d, false, sp);
  const bool fits = gr.total * 4 <= kResidentBudget;
  if (fits && 10 * worlds_per_sm(gs.total * 4) < 16 * worlds_per_sm(gr.total * 4)) {
    *g = gr, *resident = true;
    return IMN_OK;
  }
  if (gs.total * 4 > kMaxSmem)
    return set_error("imn_solve: njmax %d needs %d bytes of shared memory per world (max %d)", d->njmax,
                     gs.total * 4, kMaxSmem),
           IMN_ERR_LIMIT;
  *g = gs, *resident = false;
  return IMN_OK;
}

}  // namespace imn

#ifdef IMN_PROFILE
extern "C" int imn_debug_profile(unsigned long long* out, int reset) {
  cudaMemcpyFromSymbol(out, imn::g_prof, sizeof(unsigned long long) * 16);
  if (reset) {
    unsigned long long z[16] = {0};
    cudaMemcpyToSymbol(imn::g_prof, z, sizeof z);
  }
  return 0;
}
#endif

extern "C" int imn_set_copy_wait_limit(int32_t polls, int32_t withhold_copies) {
  if (polls <= 0) return imn::set_error("imn_set_copy_wait_limit: polls must be positive"), IMN_ERR_SHAPE;
  imn::g_wait_polls = polls;
  imn::g_withhold_copies = withhold_copies & 3;
  return IMN_OK;
}

extern "C" int imn_launch_info(const ImnModel* m, const ImnData* d, const ImnCtx* cx, ImnLaunchInfo* out) {
  if (!out) return imn::set_error("imn_launch_info: NULL out"), IMN_ERR_NULL;
  int rc = imn::validate(m, d, cx);
  if (rc) return rc;
  imn::Geom g;
  bool res;
  rc = imn::plan_launch(m, d, cx->sparse_plan, &g, &res);
  if (rc) return rc;
  out->world_threads = g.bd;
  out->worlds_per_cta = 1;
  out->smem_bytes = g.total * 4;
  out->j_resident = res ? 1 : 0;
  out->grid = d->nworld;
  return IMN_OK;
}

extern "C" int imn_solve(const ImnModel* m, const ImnData* d, const ImnCtx* cx, void* stream_) {
  int rc = imn::validate(m, d, cx);
  if (rc) return rc;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (d->nworld == 0) return IMN_OK;
  imn::Geom g;
  bool res;
  rc = imn::plan_launch(m, d, cx->sparse_plan, &g, &res);
  if (rc) return rc;
  const int bytes = g.total * 4;
  using Kernel = void (*)(ImnModel, ImnData, ImnCtx, imn::Geom, ImnSparsePlan);
  const bool sparse = cx->sparse_plan != nullptr;
  const ImnSparsePlan sp = sparse ? *cx->sparse_plan : ImnSparsePlan{};
  auto prepare = [](Kernel k, int smem) {
    // many one-warp CTAs share an SM: ask for the largest shared-memory carve-out,
    // otherwise the driver sizes it for a single CTA
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e == cudaSuccess && smem > 48 * 1024) e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    return e;
  };
  if (cx->world_order)
    imn::order_worlds_kernel<<<1, 1024, 0, stream>>>(d->nefc, d->njmax, d->nworld, cx->world_order, cx->nsolving);
  else if (cx->nsolving)
    imn::fill_nsolving<<<1, 1, 0, stream>>>(cx->nsolving, d->nworld);

  Kernel kern = sparse ? (res ? (Kernel)imn::newton_kernel_resident<true, false> : (Kernel)imn::newton_kernel_streamed<true, false>)
                       : (res ? (Kernel)imn::newton_kernel_resident<false, false> : (Kernel)imn::newton_kernel_streamed<false, false>);
  if (cx->stats)
    kern = sparse ? (res ? (Kernel)imn::newton_kernel_resident<true, true> : (Kernel)imn::newton_kernel_streamed<true, true>)
                  : (res ? (Kernel)imn::newton_kernel_resident<false, true> : (Kernel)imn::newton_kernel_streamed<false, true>);
  {
    const cudaError_t e = prepare(kern, bytes);
    if (e != cudaSuccess)
      return imn::set_error("imn_solve: cudaFuncSetAttribute: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  }
  kern<<<d->nworld, 32, bytes, stream>>>(*m, *d, *cx, g, sp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return imn::set_error("imn_solve: launch failed: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  return IMN_OK;
}
