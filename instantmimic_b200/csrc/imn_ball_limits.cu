// imn_ball_limits.cu -- directional ball-joint limit rows, appended to the constraint
// rows of every world just before the solve (reference:
// src/instantmimic/utils/mjw_kernels/ball_limits.py:36-203, launched from the constraint
// stage, src/instantmimic/utils/mjw_step_optimized.py:355-388, 2237-2249).
//
// Per limited ball joint three candidate rows: a swing ellipse in tangent-half-angle
// coordinates and the two ends of the twist interval, all functions of the joint's
// quaternion relative to its neutral pose in the anatomical frame
// (ball_limits.py:82-140; the host statement of the same residuals and Jacobians is
// ball_joint_limits.py:166-212).  A violated candidate becomes a LIMIT_JOINT row whose
// Jacobian is the residual's angular Jacobian on the joint's three dofs.
//
// The reference takes a row index with an atomic per candidate, so the order of a
// world's new rows depends on scheduling.  Here one warp owns a world, candidates
// (joint, kind) sit on lanes in ascending order and a ballot gives every violated
// candidate its rank: the rows land in (joint, kind) order, reproducibly.
//
// RESTATED: the row's impedance (efc.D, efc.aref from solref / solimp / inverse weight)
// is upstream's constraint._efc_row, whose source is not available; efc_row below
// follows MuJoCo's published solver-parameter model (spring-damper reference
// acceleration, position-dependent impedance).
#include "imn_common.cuh"

namespace imn {

struct Q4 {
  float w, x, y, z;
};
__device__ __forceinline__ Q4 qmul(Q4 a, Q4 b) {
  return Q4{a.w * b.w - (a.x * b.x + a.y * b.y + a.z * b.z),
            a.w * b.x + b.w * a.x + (a.y * b.z - a.z * b.y),
            a.w * b.y + b.w * a.y + (a.z * b.x - a.x * b.z),
            a.w * b.z + b.w * a.z + (a.x * b.y - a.y * b.x)};
}
__device__ __forceinline__ Q4 qconj(Q4 q) { return Q4{q.w, -q.x, -q.y, -q.z}; }

#define IMN_MINIMP 0.0001f
#define IMN_MAXIMP 0.9999f

// efc.D and efc.aref of one row (MuJoCo's solver parameters: solref = (time constant,
// damping ratio) or, non-positive, (-stiffness, -damping); solimp = (dmin, dmax, width,
// midpoint, power)).
__device__ __forceinline__ void efc_row(float pos, float margin, float vel, float invweight, const float* solref,
                                        const float* solimp, float timestep, bool refsafe, float& D, float& aref) {
  float timeconst = solref[0];
  const float dampratio = solref[1];
  if (refsafe) timeconst = fmaxf(timeconst, 2.0f * timestep);
  const float dmin = fminf(fmaxf(solimp[0], IMN_MINIMP), IMN_MAXIMP);
  const float dmax = fminf(fmaxf(solimp[1], IMN_MINIMP), IMN_MAXIMP);
  const float width = fmaxf(IMN_MJ_MINVAL, solimp[2]);
  const float mid = fminf(fmaxf(solimp[3], IMN_MINIMP), IMN_MAXIMP);
  const float power = fmaxf(1.0f, solimp[4]);
  float k = 1.0f / (dmax * dmax * timeconst * timeconst * dampratio * dampratio);
  float b = 2.0f / (dmax * timeconst);
  if (solref[0] <= 0.0f) k = -solref[0] / (dmax * dmax);
  if (solref[1] <= 0.0f) b = -solref[1] / dmax;
  const float x = fabsf(pos) / width;
  const float ya = (1.0f / powf(mid, power - 1.0f)) * powf(x, power);
  const float yb = 1.0f - (1.0f / powf(1.0f - mid, power - 1.0f)) * powf(1.0f - x, power);
  float imp = dmin + (x < mid ? ya : yb) * (dmax - dmin);
  imp = fminf(fmaxf(imp, dmin), dmax);
  if (x > 1.0f) imp = dmax;
  D = 1.0f / fmaxf(invweight * (1.0f - imp) / imp, IMN_MJ_MINVAL);
  aref = -k * imp * pos - b * vel;
  (void)margin;
}

// Residual r and its angular Jacobian on the joint's dofs for candidate `kind` (0 swing,
// 1 twist lower end, 2 twist upper end).  Returns false where the reference emits no
// row and counts a singular state instead (`singular` set), or no row at all.
__device__ __forceinline__ bool ball_candidate(const ImnBallLimits& P, int index, int kind, const float* qpos,
                                               float& r, float J[3], bool& singular) {
  singular = false;
  Q4 q{qpos[0], qpos[1], qpos[2], qpos[3]};
  const float qn = sqrtf(q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z);
  if (qn > 0.0f) q = Q4{q.w / qn, q.x / qn, q.y / qn, q.z / qn};
  const float* fp = P.frame + 4 * index;
  const float* np_ = P.neutral + 4 * index;
  const Q4 f{fp[0], fp[1], fp[2], fp[3]}, n{np_[0], np_[1], np_[2], np_[3]};
  q = qmul(qmul(qconj(f), qmul(qconj(n), q)), f);
  // canonical sign of the double cover
  float c[4] = {q.w, q.x, q.y, q.z};
  int pivot = 0;
  if (fabsf(c[0]) < 1.0e-15f)
    for (int k = 1; k < 4; ++k)
      if (fabsf(c[k]) > fabsf(c[pivot])) pivot = k;
  if (c[pivot] < 0.0f) q = Q4{-q.w, -q.x, -q.y, -q.z};
  const float w = q.w, x = q.x, y = q.y, z = q.z;
  const float h = w * w + z * z;
  const float minh = P.minimum_h[index];
  if (h < 0.25f * minh || fabsf(w) < 0.5f * sqrtf(minh)) {
    singular = true;  // the antipode of the swing chart: the scalar safety cap restores it
    return false;
  }
  const float sx = w * x - z * y, sy = w * y + z * x;
  float g[4];
  if (kind == 0) {
    const float* sw = P.swing + 4 * index;
    const float ax = sx < 0.0f ? sw[2] : sw[0], ay = sy < 0.0f ? sw[3] : sw[1];
    const float e = ax * sx * sx + ay * sy * sy;
    const float dh[4] = {2.0f * w, 0.0f, 0.0f, 2.0f * z};
    const float de[4] = {2.0f * ax * sx * x + 2.0f * ay * sy * y, 2.0f * ax * sx * w + 2.0f * ay * sy * z,
                         -2.0f * ax * sx * z + 2.0f * ay * sy * w, -2.0f * ax * sx * y + 2.0f * ay * sy * x};
    r = 1.0f - e / (h * h);
    for (int k = 0; k < 4; ++k) g[k] = -de[k] / (h * h) + 2.0f * e * dh[k] / (h * h * h);
  } else {
    const float theta = 2.0f * atan2f(z, w);
    g[0] = -2.0f * z / h, g[1] = 0.0f, g[2] = 0.0f, g[3] = 2.0f * w / h;
    if (kind == 1) {
      r = theta - P.twist[2 * index];
    } else {
      r = P.twist[2 * index + 1] - theta;
      for (int k = 0; k < 4; ++k) g[k] = -g[k];
    }
  }
  if (r - P.margin[index] >= 0.0f) return false;
  // angular Jacobian of g at q: 0.5 (-g0 v + w gv - v x gv), then back into joint coordinates
  const float v[3] = {x, y, z}, gv[3] = {g[1], g[2], g[3]};
  float Jl[3] = {0.5f * (-g[0] * v[0] + w * gv[0] - (v[1] * gv[2] - v[2] * gv[1])),
                 0.5f * (-g[0] * v[1] + w * gv[1] - (v[2] * gv[0] - v[0] * gv[2])),
                 0.5f * (-g[0] * v[2] + w * gv[2] - (v[0] * gv[1] - v[1] * gv[0]))};
  const float fv[3] = {f.x, f.y, f.z};
  const float t[3] = {f.w * Jl[0] + (fv[1] * Jl[2] - fv[2] * Jl[1]), f.w * Jl[1] + (fv[2] * Jl[0] - fv[0] * Jl[2]),
                      f.w * Jl[2] + (fv[0] * Jl[1] - fv[1] * Jl[0])};
  J[0] = Jl[0] + 2.0f * (fv[1] * t[2] - fv[2] * t[1]);
  J[1] = Jl[1] + 2.0f * (fv[2] * t[0] - fv[0] * t[2]);
  J[2] = Jl[2] + 2.0f * (fv[0] * t[1] - fv[1] * t[0]);
  if (J[0] * J[0] + J[1] * J[1] + J[2] * J[2] < 1.0e-16f) {
    singular = true;
    return false;
  }
  return true;
}

static const int kBallWarps = 4;

__global__ void __launch_bounds__(32 * kBallWarps) ball_limit_kernel(const ImnBallLimits P, const int nworld) {
  const int lane = threadIdx.x & 31, w = blockIdx.x * kBallWarps + (threadIdx.x >> 5);
  if (w >= nworld) return;
  const int ncand = 3 * P.njoint;
  int base = P.nefc[w], added = 0, lost = 0, nsing = 0;
#pragma unroll 1
  for (int c0 = 0; c0 < ncand; c0 += 32) {
    const int c = c0 + lane;
    bool active = false, singular = false;
    float r = 0.0f, J[3] = {0.0f, 0.0f, 0.0f};
    int index = 0;
    if (c < ncand) {
      index = c / 3;
      active = ball_candidate(P, index, c - 3 * index, P.qpos + (size_t)w * P.qpos_ld + P.qadr[index], r, J, singular);
    }
    const unsigned am = __ballot_sync(IMN_FULL_MASK, active);
    nsing += __popc(__ballot_sync(IMN_FULL_MASK, singular));
    if (active) {
      const int efcid = base + added + __popc(am & ((1u << lane) - 1u));
      if (efcid < P.njmax) {
        const int dof = P.dadr[index];
        float* Jr = P.efc_J + (size_t)w * P.J_ld_world + (size_t)efcid * P.J_ld_row;
        for (int k = 0; k < P.nv; ++k) Jr[k] = 0.0f;
        for (int k = 0; k < 3; ++k) Jr[dof + k] = J[k];
        const float* qv = P.qvel + (size_t)w * P.qvel_ld + dof;
        const float vel = J[0] * qv[0] + J[1] * qv[1] + J[2] * qv[2];
        const float jn = J[0] * J[0] + J[1] * J[1] + J[2] * J[2];
        // the native ball row's scalar inverse weight, scaled by this Jacobian's squared norm
        const float weight = P.invweight[(size_t)(w % P.n_invweight) * P.nv + dof] * jn;
        const float margin = P.margin[index], pos = r - margin;
        float D, aref;
        efc_row(pos, margin, vel, weight, P.solref + 2 * index, P.solimp + 5 * index, P.timestep[w % P.n_timestep], P.refsafe != 0, D,
                aref);
        const size_t o = (size_t)w * P.efc_ld + efcid;
        P.efc_type[o] = P.limit_joint_type;
        P.efc_id[o] = P.joint[index];
        P.efc_pos[o] = pos + margin;
        P.efc_margin[o] = margin;
        P.efc_D[o] = D;
        P.efc_vel[o] = vel;
        P.efc_aref[o] = aref;
        P.efc_frictionloss[o] = 0.0f;
      }
    }
    added += __popc(am);
  }
  lost = max(0, base + added - P.njmax) - max(0, base - P.njmax);
  if (lane == 0) {
    P.nefc[w] = base + added;
    if (P.nl) P.nl[w] += added;
    if (P.overflow && lost > 0) P.overflow[w] += lost;
    if (P.singular && nsing > 0) P.singular[w] += nsing;
  }
}

}  // namespace imn

extern "C" int imn_ball_limit_rows(const ImnBallLimits* p, int32_t nworld, void* stream) {
  if (!p) return imn::set_error("imn_ball_limit_rows: NULL struct"), IMN_ERR_NULL;
  const void* need[] = {p->qadr,   p->dadr,     p->joint,   p->neutral,   p->frame,      p->swing,   p->twist,
                        p->minimum_h, p->margin, p->solref,  p->solimp,    p->invweight,  p->qpos,    p->qvel,
                        p->nefc,   p->efc_type, p->efc_id,  p->efc_J,     p->efc_pos,    p->efc_margin, p->efc_D,
                        p->efc_vel, p->efc_aref, p->efc_frictionloss, p->timestep};
  for (const void* q : need)
    if (!q) return imn::set_error("imn_ball_limit_rows: a required pointer is NULL"), IMN_ERR_NULL;
  if (p->njoint < 0 || p->nv <= 0 || p->njmax < 0 || nworld < 0 || p->n_invweight <= 0 || p->n_timestep <= 0 || p->J_ld_row < p->nv ||
      p->efc_ld < p->njmax || p->J_ld_world < (int64_t)p->njmax * p->J_ld_row)
    return imn::set_error("imn_ball_limit_rows: bad extent or stride"), IMN_ERR_SHAPE;
  if (p->njmax < 3 * p->njoint)
    return imn::set_error("imn_ball_limit_rows: directional ball constraints need three reserved rows per joint "
                          "(njmax %d, %d joints)", p->njmax, p->njoint),
           IMN_ERR_LIMIT;
  if (nworld == 0 || p->njoint == 0) return IMN_OK;
  imn::ball_limit_kernel<<<(nworld + imn::kBallWarps - 1) / imn::kBallWarps, 32 * imn::kBallWarps, 0,
                           (cudaStream_t)stream>>>(*p, nworld);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return imn::set_error("imn_ball_limit_rows: launch failed: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  return IMN_OK;
}
