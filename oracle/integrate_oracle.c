/* integrate_oracle.c -- CPU statement of the implicit-fast integrator's tail
 * (reference: _integrate, src/instantmimic/utils/mjw_step_optimized.py:5209-5297).
 *
 * TEST INFRASTRUCTURE: used by tests/ only, never by the product path.
 *
 * oracle_implicit_matrix: A = M - h qDeriv on M's CSR entries, qDeriv = actuator term
 *   sum_a moment_a moment_a^T gain_a (mjw_step_optimized.py:629-669: pairs rowj <= rowi
 *   of each actuator's moment row land on M_elemid[dofi, dofj]) minus diag(dof_damping)
 *   (upstream derivative._qderiv_actuator_passive).  RESTATED: the upstream kernels are
 *   not available; the reference itself accumulates the actuator products with atomics,
 *   so its summation order is not defined.  Here every entry takes its products in
 *   ascending actuator order.
 * oracle_advance: qvel += h qacc, qpos integrated with the new qvel, time += h
 *   (upstream _advance through _advance_with_scratch, :4823-4847).  RESTATED from
 *   MuJoCo's mj_advance / mju_quatIntegrate.
 * Parity unpinned against the reference for both (no reference run, no golden vector).
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "../include/imnewton.h"
#include "oracle_common.h"

int oracle_implicit_matrix(const ImnImplicit* p, const float* M, int64_t M_ld, float* out, int64_t out_ld,
                           int nworld) {
  float* qd = (float*)malloc(sizeof(float) * (size_t)p->nM);
  for (int w = 0; w < nworld; ++w) {
    memset(qd, 0, sizeof(float) * (size_t)p->nM);
    if (p->nu > 0 && p->actuation) {
      const int32_t* rownnz = p->moment_rownnz + (size_t)w * p->nu;
      const int32_t* rowadr = p->moment_rowadr + (size_t)w * p->nu;
      const int32_t* colind = p->moment_colind + (size_t)w * p->moment_ld;
      const float* moment = p->actuator_moment + (size_t)w * p->moment_ld;
      const float* gain = p->actuator_velocity_gain + (size_t)w * p->nu;
      for (int a = 0; a < p->nu; ++a) {
        const float vel = gain[a];
        if (vel == 0.0f) continue;
        for (int ri = 0; ri < rownnz[a]; ++ri)
          for (int rj = 0; rj <= ri; ++rj) {
            const int di = colind[rowadr[a] + ri], dj = colind[rowadr[a] + rj];
            const int e = p->M_elemid[di * p->nv + dj];
            if (e < 0) continue;
            const float c = (moment[rowadr[a] + ri] * moment[rowadr[a] + rj]) * vel;
            if (c != 0.0f) qd[e] = qd[e] + c;
          }
      }
    }
    if (p->damper)
      for (int i = 0; i < p->nv; ++i) {
        const int e = p->M_elemid[i * p->nv + i];
        qd[e] = qd[e] - p->dof_damping[i];
      }
    for (int e = 0; e < p->nM; ++e) out[(size_t)w * out_ld + e] = M[(size_t)w * M_ld + e] - p->timestep[w % p->n_timestep] * qd[e];
  }
  free(qd);
  return 0;
}

static void quat_integrate(float q[4], const float w[3], float h) {
  const float norm = sqrtf(w[0] * w[0] + w[1] * w[1] + w[2] * w[2]);
  float r[4] = {1.0f, 0.0f, 0.0f, 0.0f};
  if (norm >= MJ_MINVAL) {
    const float half = 0.5f * (h * norm);
    const float s = sinf(half) / norm;
    r[0] = cosf(half), r[1] = w[0] * s, r[2] = w[1] * s, r[3] = w[2] * s;
  }
  const float a = q[0], b = q[1], c = q[2], d = q[3];
  float o[4] = {a * r[0] - b * r[1] - c * r[2] - d * r[3], a * r[1] + b * r[0] + c * r[3] - d * r[2],
                a * r[2] - b * r[3] + c * r[0] + d * r[1], a * r[3] + b * r[2] - c * r[1] + d * r[0]};
  const float len = sqrtf(o[0] * o[0] + o[1] * o[1] + o[2] * o[2] + o[3] * o[3]);
  if (len < MJ_MINVAL) {
    q[0] = 1.0f, q[1] = q[2] = q[3] = 0.0f;
    return;
  }
  const float inv = 1.0f / len;
  for (int k = 0; k < 4; ++k) q[k] = o[k] * inv;
}

int oracle_advance(const ImnAdvance* p, const float* qacc, int64_t qacc_ld, int nworld) {
  for (int w = 0; w < nworld; ++w) {
    const float h = p->timestep[w % p->n_timestep];
    for (int j = 0; j < p->njnt; ++j) {
      const int type = p->jnt_type[j], dof = p->jnt_dofadr[j], pos = p->jnt_qposadr[j];
      float* qvel = p->qvel + (size_t)w * p->qvel_ld + dof;
      float* qpos = p->qpos + (size_t)w * p->qpos_ld + pos;
      const float* acc = qacc + (size_t)w * qacc_ld + dof;
      const int ndof = type == IMN_JNT_FREE ? 6 : (type == IMN_JNT_BALL ? 3 : 1);
      float v[6];
      for (int k = 0; k < ndof; ++k) {
        v[k] = qvel[k] + h * acc[k];
        qvel[k] = v[k];
      }
      if (type == IMN_JNT_FREE) {
        for (int k = 0; k < 3; ++k) qpos[k] = qpos[k] + h * v[k];
        quat_integrate(qpos + 3, v + 3, h);
      } else if (type == IMN_JNT_BALL) {
        quat_integrate(qpos, v, h);
      } else {
        qpos[0] = qpos[0] + h * v[0];
      }
    }
    if (p->time) p->time[w] = p->time[w] + h;
  }
  return 0;
}
