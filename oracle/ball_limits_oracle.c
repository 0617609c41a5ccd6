/* ball_limits_oracle.c -- CPU statement of the directional ball-joint limit rows
 * (reference: src/instantmimic/utils/mjw_kernels/ball_limits.py:36-203).
 *
 * TEST INFRASTRUCTURE: used by tests/ only, never by the product path.
 *
 * Geometry (residuals, Jacobians): follows ball_limits.py:82-140 and is pinned against
 * the reference's own host function limit_residuals (ball_joint_limits.py:166-212)
 * through tests/golden/ball_limit_reference.npz.
 * Row impedance (efc.D, efc.aref): RESTATED -- upstream constraint._efc_row is not
 * available; efc_row follows MuJoCo's published solver-parameter model.  Unpinned.
 * Row order: candidates in ascending (joint, kind) order (the reference's order
 * depends on its atomics).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>

#include "../include/imnewton.h"
#include "oracle_common.h"

typedef struct {
  float w, x, y, z;
} Q4;
static Q4 qmul(Q4 a, Q4 b) {
  Q4 o = {a.w * b.w - (a.x * b.x + a.y * b.y + a.z * b.z), a.w * b.x + b.w * a.x + (a.y * b.z - a.z * b.y),
          a.w * b.y + b.w * a.y + (a.z * b.x - a.x * b.z), a.w * b.z + b.w * a.z + (a.x * b.y - a.y * b.x)};
  return o;
}
static Q4 qconj(Q4 q) {
  Q4 o = {q.w, -q.x, -q.y, -q.z};
  return o;
}
static float clampf(float v, float lo, float hi) { return fminf(fmaxf(v, lo), hi); }

static void efc_row(float pos, float vel, float invweight, const float* solref, const float* solimp, float timestep,
                    int refsafe, float* D, float* aref) {
  float timeconst = solref[0];
  const float dampratio = solref[1];
  if (refsafe) timeconst = fmaxf(timeconst, 2.0f * timestep);
  const float dmin = clampf(solimp[0], 0.0001f, 0.9999f), dmax = clampf(solimp[1], 0.0001f, 0.9999f);
  const float width = fmaxf(MJ_MINVAL, solimp[2]);
  const float mid = clampf(solimp[3], 0.0001f, 0.9999f);
  const float power = fmaxf(1.0f, solimp[4]);
  float k = 1.0f / (dmax * dmax * timeconst * timeconst * dampratio * dampratio);
  float b = 2.0f / (dmax * timeconst);
  if (solref[0] <= 0.0f) k = -solref[0] / (dmax * dmax);
  if (solref[1] <= 0.0f) b = -solref[1] / dmax;
  const float x = fabsf(pos) / width;
  const float ya = (1.0f / powf(mid, power - 1.0f)) * powf(x, power);
  const float yb = 1.0f - (1.0f / powf(1.0f - mid, power - 1.0f)) * powf(1.0f - x, power);
  float imp = dmin + (x < mid ? ya : yb) * (dmax - dmin);
  imp = clampf(imp, dmin, dmax);
  if (x > 1.0f) imp = dmax;
  *D = 1.0f / fmaxf(invweight * (1.0f - imp) / imp, MJ_MINVAL);
  *aref = -k * imp * pos - b * vel;
}

/* 1: row, 0: none, -1: singular */
static int candidate(const ImnBallLimits* P, int index, int kind, const float* qpos, float* r_out, float J[3]) {
  Q4 q = {qpos[0], qpos[1], qpos[2], qpos[3]};
  const float qn = sqrtf(q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z);
  if (qn > 0.0f) q.w /= qn, q.x /= qn, q.y /= qn, q.z /= qn;
  const float *fp = P->frame + 4 * index, *np_ = P->neutral + 4 * index;
  const Q4 f = {fp[0], fp[1], fp[2], fp[3]}, n = {np_[0], np_[1], np_[2], np_[3]};
  q = qmul(qmul(qconj(f), qmul(qconj(n), q)), f);
  float c[4] = {q.w, q.x, q.y, q.z};
  int pivot = 0;
  if (fabsf(c[0]) < 1.0e-15f)
    for (int k = 1; k < 4; ++k)
      if (fabsf(c[k]) > fabsf(c[pivot])) pivot = k;
  if (c[pivot] < 0.0f) q.w = -q.w, q.x = -q.x, q.y = -q.y, q.z = -q.z;
  const float w = q.w, x = q.x, y = q.y, z = q.z;
  const float h = w * w + z * z, minh = P->minimum_h[index];
  if (h < 0.25f * minh || fabsf(w) < 0.5f * sqrtf(minh)) return -1;
  const float sx = w * x - z * y, sy = w * y + z * x;
  float g[4], r;
  if (kind == 0) {
    const float* sw = P->swing + 4 * index;
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
      r = theta - P->twist[2 * index];
    } else {
      r = P->twist[2 * index + 1] - theta;
      for (int k = 0; k < 4; ++k) g[k] = -g[k];
    }
  }
  *r_out = r;
  if (r - P->margin[index] >= 0.0f) return 0;
  const float v[3] = {x, y, z}, gv[3] = {g[1], g[2], g[3]};
  const float Jl[3] = {0.5f * (-g[0] * v[0] + w * gv[0] - (v[1] * gv[2] - v[2] * gv[1])),
                       0.5f * (-g[0] * v[1] + w * gv[1] - (v[2] * gv[0] - v[0] * gv[2])),
                       0.5f * (-g[0] * v[2] + w * gv[2] - (v[0] * gv[1] - v[1] * gv[0]))};
  const float fv[3] = {f.x, f.y, f.z};
  const float t[3] = {f.w * Jl[0] + (fv[1] * Jl[2] - fv[2] * Jl[1]), f.w * Jl[1] + (fv[2] * Jl[0] - fv[0] * Jl[2]),
                      f.w * Jl[2] + (fv[0] * Jl[1] - fv[1] * Jl[0])};
  J[0] = Jl[0] + 2.0f * (fv[1] * t[2] - fv[2] * t[1]);
  J[1] = Jl[1] + 2.0f * (fv[2] * t[0] - fv[0] * t[2]);
  J[2] = Jl[2] + 2.0f * (fv[0] * t[1] - fv[1] * t[0]);
  if (J[0] * J[0] + J[1] * J[1] + J[2] * J[2] < 1.0e-16f) return -1;
  return 1;
}

int oracle_ball_limit_rows(const ImnBallLimits* P, int nworld) {
  for (int w = 0; w < nworld; ++w) {
    const int base = P->nefc[w];
    int added = 0, nsing = 0;
    for (int index = 0; index < P->njoint; ++index)
      for (int kind = 0; kind < 3; ++kind) {
        float r, J[3];
        const int got = candidate(P, index, kind, P->qpos + (size_t)w * P->qpos_ld + P->qadr[index], &r, J);
        if (got < 0) ++nsing;
        if (got <= 0) continue;
        const int efcid = base + added++;
        if (efcid >= P->njmax) continue;
        const int dof = P->dadr[index];
        float* Jr = P->efc_J + (size_t)w * P->J_ld_world + (size_t)efcid * P->J_ld_row;
        for (int k = 0; k < P->nv; ++k) Jr[k] = 0.0f;
        for (int k = 0; k < 3; ++k) Jr[dof + k] = J[k];
        const float* qv = P->qvel + (size_t)w * P->qvel_ld + dof;
        const float vel = J[0] * qv[0] + J[1] * qv[1] + J[2] * qv[2];
        const float jn = J[0] * J[0] + J[1] * J[1] + J[2] * J[2];
        const float weight = P->invweight[(size_t)(w % P->n_invweight) * P->nv + dof] * jn;
        const float margin = P->margin[index], pos = r - margin;
        float D, aref;
        efc_row(pos, vel, weight, P->solref + 2 * index, P->solimp + 5 * index, P->timestep[w % P->n_timestep], P->refsafe, &D, &aref);
        const size_t o = (size_t)w * P->efc_ld + efcid;
        P->efc_type[o] = P->limit_joint_type, P->efc_id[o] = P->joint[index];
        P->efc_pos[o] = pos + margin, P->efc_margin[o] = margin;
        P->efc_D[o] = D, P->efc_vel[o] = vel, P->efc_aref[o] = aref, P->efc_frictionloss[o] = 0.0f;
      }
    P->nefc[w] = base + added;
    if (P->nl) P->nl[w] += added;
    const int lost = (base + added > P->njmax ? base + added - P->njmax : 0) - (base > P->njmax ? base - P->njmax : 0);
    if (P->overflow && lost > 0) P->overflow[w] += lost;
    if (P->singular && nsing > 0) P->singular[w] += nsing;
  }
  return 0;
}
