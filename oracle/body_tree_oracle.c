/* body_tree_oracle.c -- CPU statement of the body-tree reductions and the stages built on
 * them (reference: src/instantmimic/utils/mjw_kernels/tree_fusion.py, velocity_fusion.py).
 *
 * TEST INFRASTRUCTURE: used by tests/ only, never by the product path.
 *
 * oracle_body_tree_accumulate: the depth-ordered sum of tree_fusion.py:80-112 -- levels
 *   from the deepest up, bodies of a level in list order, parent += child.  PINNED: the
 *   reference's own tests state this sum as a plain loop and require its deterministic
 *   kernels to equal it bit for bit (tests/test_mjw_tree_fusion.py:36-41, 142-160); the
 *   same loops and the same golden cancellation case are in this repository's tests.
 * oracle_crb / oracle_rne: tree_fusion.py:186-222.  RESTATED: the per-body arithmetic is
 *   upstream mujoco-warp (smooth._M, _rne_cacc_*, _rne_cfrc, _qfrc_bias, math.inert_vec,
 *   math.motion_cross_force), not available here; this is MuJoCo's published mj_crb /
 *   mj_rne arithmetic with every sum a left-to-right fused multiply-add chain.  Parity
 *   unpinned against the reference (the reference's own test allows 1e-5 between its
 *   fused and upstream paths, tests/test_mjw_tree_fusion.py:131-134).
 * oracle_com_vel: velocity_fusion.py:15-103, joint branch by joint branch; motion_cross
 *   RESTATED from MuJoCo's mju_crossMotion.  Parity unpinned.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "../include/imnewton.h"
#include "oracle_common.h"

static void sweep_up(const ImnBodyTree* T, float* v, int C, int skip_root_parent) {
  for (int level = T->nlevels - 1; level >= 0; --level)
    for (int pos = T->level_offsets[level]; pos < T->level_offsets[level + 1]; ++pos) {
      const int body = T->level_bodies[pos], parent = T->body_parentid[body];
      if (body != 0 && (!skip_root_parent || parent != 0))
        for (int c = 0; c < C; ++c) v[parent * C + c] = v[parent * C + c] + v[body * C + c];
    }
}

int oracle_body_tree_accumulate(const ImnBodyTree* T, float* values, int64_t world_ld, int components,
                                int skip_root_parent, int nworld) {
  for (int w = 0; w < nworld; ++w) sweep_up(T, values + (size_t)w * world_ld, components, skip_root_parent);
  return 0;
}

static float dot6(const float* a, const float* b) {
  float acc = a[0] * b[0];
  for (int k = 1; k < 6; ++k) acc = fmaf(a[k], b[k], acc);
  return acc;
}
static float det2(float x, float yp, float y, float xp) { return fmaf(x, yp, -(y * xp)); }
static void cross3(const float* a, const float* b, float* r) {
  r[0] = det2(a[1], b[2], a[2], b[1]);
  r[1] = det2(a[2], b[0], a[0], b[2]);
  r[2] = det2(a[0], b[1], a[1], b[0]);
}
static void motion_cross(const float* vel, const float* a, float* r) {
  float t[3], u[3];
  cross3(vel, a, r);
  cross3(vel, a + 3, t);
  cross3(vel + 3, a, u);
  for (int k = 0; k < 3; ++k) r[3 + k] = t[k] + u[k];
}
static void motion_cross_force(const float* vel, const float* f, float* r) {
  float t[3], u[3];
  cross3(vel, f, t);
  cross3(vel + 3, f + 3, u);
  for (int k = 0; k < 3; ++k) r[k] = t[k] + u[k];
  cross3(vel, f + 3, r + 3);
}
static void inert_vec(const float* i, const float* v, float* r) {
  r[0] = fmaf(i[7], v[5], fmaf(-i[8], v[4], fmaf(i[4], v[2], fmaf(i[0], v[0], i[3] * v[1]))));
  r[1] = fmaf(-i[6], v[5], fmaf(i[8], v[3], fmaf(i[5], v[2], fmaf(i[3], v[0], i[1] * v[1]))));
  r[2] = fmaf(i[6], v[4], fmaf(-i[7], v[3], fmaf(i[2], v[2], fmaf(i[4], v[0], i[5] * v[1]))));
  r[3] = fmaf(i[9], v[3], fmaf(i[8], v[1], -(i[7] * v[2])));
  r[4] = fmaf(i[9], v[4], fmaf(i[6], v[2], -(i[8] * v[0])));
  r[5] = fmaf(i[9], v[5], fmaf(i[7], v[0], -(i[6] * v[1])));
}
static void axpy6(float* a, const float* b, float s) {
  for (int k = 0; k < 6; ++k) a[k] = fmaf(b[k], s, a[k]);
}

int oracle_crb(const ImnBodyTree* T, const float* cinert, const float* cdof, float* crb, float* M, int64_t M_ld,
               int nworld) {
  for (int w = 0; w < nworld; ++w) {
    float* c = crb + (size_t)w * T->nbody * 10;
    const float* dof = cdof + (size_t)w * T->nv * 6;
    memcpy(c, cinert + (size_t)w * T->nbody * 10, sizeof(float) * (size_t)T->nbody * 10);
    sweep_up(T, c, 10, 1);
    const float* arm = T->dof_armature + (size_t)(w % T->n_armature) * T->nv;
    float* Mw = M + (size_t)w * M_ld;
    for (int i = 0; i < T->nv; ++i) {
      float buf[6];
      inert_vec(c + 10 * T->dof_bodyid[i], dof + 6 * i, buf);
      /* row i of M: the ancestors of i in ascending order, the diagonal last
       * (tree_fusion.py:192-206 hands upstream's kernel M_rownnz / M_rowadr; here the
       * row's end is found from the entry table) */
      int adr = -1;
      for (int e = 0; e < T->nM; ++e)
        if (T->M_rowidx[e] == i && T->M_colind[e] == i) adr = e;
      Mw[adr] = arm[i] + dot6(dof + 6 * i, buf);
      for (int j = T->dof_parentid[i]; j >= 0; j = T->dof_parentid[j]) Mw[--adr] = dot6(dof + 6 * j, buf);
    }
  }
  return 0;
}

int oracle_rne(const ImnBodyTree* T, const float* cinert, const float* cvel, const float* cdof, const float* cdof_dot,
               const float* qvel, int64_t qvel_ld, float* cacc, float* cfrc_int, float* qfrc_bias, int64_t bias_ld,
               int nworld) {
  for (int w = 0; w < nworld; ++w) {
    float* a = cacc + (size_t)w * T->nbody * 6;
    float* f = cfrc_int + (size_t)w * T->nbody * 6;
    const float* dd = cdof_dot + (size_t)w * T->nv * 6;
    const float* dof = cdof + (size_t)w * T->nv * 6;
    const float* qv = qvel + (size_t)w * qvel_ld;
    const float* g = T->gravity + 3 * (size_t)(w % T->n_gravity);
    for (int k = 0; k < 6; ++k) a[k] = (k < 3 || !T->gravity_enabled) ? 0.0f : -g[k - 3], f[k] = 0.0f;
    for (int level = 1; level < T->nlevels; ++level)
      for (int pos = T->level_offsets[level]; pos < T->level_offsets[level + 1]; ++pos) {
        const int b = T->level_bodies[pos];
        float acc[6];
        memcpy(acc, a + 6 * T->body_parentid[b], sizeof acc);
        for (int d = T->body_dofadr[b]; d < T->body_dofadr[b] + T->body_dofnum[b]; ++d) axpy6(acc, dd + 6 * d, qv[d]);
        memcpy(a + 6 * b, acc, sizeof acc);
      }
    for (int b = 1; b < T->nbody; ++b) {
      const float* I = cinert + ((size_t)w * T->nbody + b) * 10;
      const float* v = cvel + ((size_t)w * T->nbody + b) * 6;
      float fa[6], iv[6], x[6];
      inert_vec(I, a + 6 * b, fa);
      inert_vec(I, v, iv);
      motion_cross_force(v, iv, x);
      for (int k = 0; k < 6; ++k) f[6 * b + k] = fa[k] + x[k];
    }
    sweep_up(T, f, 6, 0);
    for (int i = 0; i < T->nv; ++i) qfrc_bias[(size_t)w * bias_ld + i] = dot6(dof + 6 * i, f + 6 * T->dof_bodyid[i]);
  }
  return 0;
}

int oracle_com_vel(const ImnBodyTree* T, const float* qvel, int64_t qvel_ld, const float* cdof, float* cvel,
                   float* cdof_dot, int nworld) {
  for (int w = 0; w < nworld; ++w) {
    float* cv = cvel + (size_t)w * T->nbody * 6;
    float* dot = cdof_dot + (size_t)w * T->nv * 6;
    const float* dof = cdof + (size_t)w * T->nv * 6;
    const float* qv = qvel + (size_t)w * qvel_ld;
    for (int level = 0; level < T->nlevels; ++level)
      for (int pos = T->level_offsets[level]; pos < T->level_offsets[level + 1]; ++pos) {
        const int b = T->level_bodies[pos];
        float v[6] = {0};
        if (b != 0) {
          memcpy(v, cv + 6 * T->body_parentid[b], sizeof v);
          int d = T->body_dofadr[b];
          for (int j = T->body_jntadr[b]; j < T->body_jntadr[b] + T->body_jntnum[b]; ++j) {
            const int type = T->jnt_type[j];
            if (type == IMN_JNT_FREE) {
              for (int k = 0; k < 3; ++k) {
                axpy6(v, dof + 6 * (d + k), qv[d + k]);
                memset(dot + 6 * (d + k), 0, 6 * sizeof(float));
              }
              for (int k = 3; k < 6; ++k) motion_cross(v, dof + 6 * (d + k), dot + 6 * (d + k));
              for (int k = 3; k < 6; ++k) axpy6(v, dof + 6 * (d + k), qv[d + k]);
              d += 6;
            } else if (type == IMN_JNT_BALL) {
              for (int k = 0; k < 3; ++k) motion_cross(v, dof + 6 * (d + k), dot + 6 * (d + k));
              for (int k = 0; k < 3; ++k) axpy6(v, dof + 6 * (d + k), qv[d + k]);
              d += 3;
            } else {
              motion_cross(v, dof + 6 * d, dot + 6 * d);
              axpy6(v, dof + 6 * d, qv[d]);
              d += 1;
            }
          }
        }
        memcpy(cv + 6 * b, v, sizeof v);
      }
  }
  return 0;
}
