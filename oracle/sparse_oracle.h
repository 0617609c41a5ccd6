/* sparse_oracle.h -- prototypes of sparse_oracle.c.  TEST INFRASTRUCTURE ONLY. */
#ifndef SPARSE_ORACLE_H_
#define SPARSE_ORACLE_H_
#include "../include/imnewton.h"
void sparse_factor_levels(const ImnSparsePlan* P, float* N, float* iD);
void sparse_load_rhs(const ImnSparsePlan* P, float* N, const float* grad);
void sparse_forward(const ImnSparsePlan* P, float* N, const float* iD, const float* grad);
void sparse_backward(const ImnSparsePlan* P, float* N, const float* iD, const float* grad, float* search,
                     int bd, float sums[2]);
int sparse_assemble(const ImnSparsePlan* P, float* N, const float* M, const float* J, int ldj,
                    const float* D, const int* state, int nefc);
int sparse_update(const ImnSparsePlan* P, float* Hp, const float* J, int ldj, const float* D, const int* state,
                  const int* ids, int count, const int* uni, int n);
#endif
