"""Builds oracle/_ref/libref_snippets.so: the REFERENCE'S OWN CUDA text, compiled with nvcc.

TEST INFRASTRUCTURE.  Nothing here is imported by the product path; only tests/ and the
build step of the repository's entry script use it.

The reference writes the numeric core of two stages of the solve as CUDA source strings
that it hands to Warp's native-function hook:

* the sparse-pattern Hessian factor (``sparse_hessian.build_plan``,
  src/instantmimic/utils/mjw_kernels/sparse_hessian.py:229-702): ``init_snippet`` (initial
  assembly H = M + J'DJ on the pattern, factor, solve), ``factor_snippet`` (incremental H
  update + refactor + solve, solve with the resident factor) and ``nonfused_snippet``
  (factor of the dense upstream H, solve);
* the tree L'DL factor/solve of M (``tree_ldl._generate_source``, tree_ldl.py:194-383).

Those strings need nothing of Warp but its array accessor and a two-float return type, so
they compile as they are once a twenty-line stand-in provides ``wp::address`` and
``wp::vec2``.  This script imports the two reference modules from the reference tree (with
empty stand-ins for the modules they name at import time but do not call on this path),
asks them for the generated text of a few models, wraps every snippet in a function of the
signature the reference declares for it (sparse_hessian.py:761-779, 809-821, 858-866;
tree_ldl.py:388-396), adds kernels that call those functions the way the reference's Warp
kernels do (sparse_hessian.py:823-844, 870-892; tree_ldl.py:398-404, 428-433) and compiles
the lot with nvcc's defaults -- fused multiply-add contraction ON, as Warp compiles its
modules -- for sm_100a.

Everything it writes goes to oracle/_ref/ (git-ignored): the generated .cu holds reference
text and is never committed.  The reference tree is needed only to BUILD; the library and
the golden vectors made from it (tests/golden/make_ref_snippet_golden.py) work without it.

    python -m oracle.ref_snippets [reference root]
"""

from __future__ import annotations

import enum
import importlib.util
import json
import subprocess
import sys
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
LIB = OUT / "libref_snippets.so"
MANIFEST = OUT / "ref_snippets.json"

sys.path.insert(0, str(HERE.parent))

SHIM = r"""
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
// What the snippets use of Warp: element addresses of arrays, shape[], a two-float value.
namespace wp {
struct vec2 {
  float c[2];
  __device__ vec2(float a = 0.0f, float b = 0.0f) { c[0] = a; c[1] = b; }
  __device__ float operator[](int i) const { return c[i]; }
};
template <class T> struct arr {
  T* data;
  int shape[3];
  long long strides[3];  // in elements
};
template <class T> __device__ T* address(const arr<T>& a, int i) { return a.data + i * a.strides[0]; }
template <class T> __device__ T* address(const arr<T>& a, int i, int j) { return a.data + i * a.strides[0] + j * a.strides[1]; }
template <class T> __device__ T* address(const arr<T>& a, int i, int j, int k) {
  return a.data + i * a.strides[0] + j * a.strides[1] + k * a.strides[2];
}
}  // namespace wp
typedef wp::arr<float> fa;
typedef wp::arr<int> ia;
// world w of a (W, n) array as an (n, 1) array, as `a[w]` of a reshaped (W, n, 1) Warp array
__device__ inline fa row_of(const float* p, long long ld, int n, int w) {
  fa a; a.data = const_cast<float*>(p) + (long long)w * ld; a.shape[0] = n; a.shape[1] = 1; a.shape[2] = 1;
  a.strides[0] = 1; a.strides[1] = 1; a.strides[2] = 0; return a;
}
// world w of a (W, P, P) array as a (P, P) array
__device__ inline fa mat_of(const float* p, int P, int w) {
  fa a; a.data = const_cast<float*>(p) + (long long)w * P * P; a.shape[0] = P; a.shape[1] = P; a.shape[2] = 1;
  a.strides[0] = P; a.strides[1] = 1; a.strides[2] = 0; return a;
}
template <class T> inline wp::arr<T> make2(const T* p, int n0, int n1) {
  wp::arr<T> a; a.data = const_cast<T*>(p); a.shape[0] = n0; a.shape[1] = n1; a.shape[2] = 1;
  a.strides[0] = n1; a.strides[1] = 1; a.strides[2] = 0; return a;
}
template <class T> inline wp::arr<T> make3(const T* p, int n0, int n1, int n2) {
  wp::arr<T> a; a.data = const_cast<T*>(p); a.shape[0] = n0; a.shape[1] = n1; a.shape[2] = n2;
  a.strides[0] = (long long)n1 * n2; a.strides[1] = n2; a.strides[2] = 1; return a;
}
"""

CASE = r"""
namespace case_@NAME@ {
// ---- fused plan (block @FB@) ------------------------------------------------------------
__device__ wp::vec2 sparse_newton_native(fa J, fa D, ia state, ia ids, int count, ia uni, int w, fa Hd, fa grad, fa U,
                                         fa search, int lane_in, int mode) {
@FACTOR@
}
__device__ wp::vec2 sparse_newton_init_native(fa J, fa D, ia state, int nefc_in, fa M, int w, fa grad, fa U, fa search,
                                              int lane_in) {
@INIT@
}
__global__ void k_init(const unsigned char* done, const int* nefc, fa J, fa D, ia state, fa M, const float* grad,
                       int grad_ld, float* U, float* search, float* search_dot, float* decrement) {
  const int w = blockIdx.x, lane = threadIdx.x;
  if (done[w]) return;
  const wp::vec2 sums = sparse_newton_init_native(J, D, state, nefc[w], M, w, row_of(grad, grad_ld, grad_ld, w),
                                                  mat_of(U, @P@, w), row_of(search, @NV@, @NV@, w), lane);
  if (lane == 0) search_dot[w] = sums[0], decrement[w] = sums[1];
}
// mode 0: incremental update + refactor + solve; mode 1: the factor is loaded from U into
// the block (the reference's mode 2) and the solve with the resident factor runs
__global__ void k_fused(fa J, fa D, ia state, ia ids, const int* count, ia uni, const float* grad, int grad_ld, float* U,
                        float* search, float* search_dot, float* decrement, int mode) {
  const int w = blockIdx.x, lane = threadIdx.x;
  fa none; none.data = nullptr;
  const fa g = row_of(grad, grad_ld, grad_ld, w), u = mat_of(U, @P@, w), s = row_of(search, @NV@, @NV@, w);
  if (mode == 1) sparse_newton_native(J, D, state, ids, 0, uni, w, none, g, u, s, lane, 2);
  const wp::vec2 sums = sparse_newton_native(J, D, state, ids, count[w], uni, w, none, g, u, s, lane, mode);
  if (lane == 0) search_dot[w] = sums[0], decrement[w] = sums[1];
}
// ---- non-fused plan (block @NB@) -----------------------------------------------------------
__device__ wp::vec2 sparse_newton_upstream_native(fa Hd, fa grad, fa U, fa search, int lane_in, int mode) {
@NONFUSED@
}
__global__ void k_nonfused(const unsigned char* done, const float* grad, int grad_ld, const float* H,
                           const int* quad_changed, const int* state_changed, float* U, float* search,
                           float* search_dot, float* decrement, int skip_unchanged, int skip_noflip) {
  const int w = blockIdx.x, lane = threadIdx.x;
  if (done[w]) return;
  if (skip_noflip && state_changed[w] == 0) return;
  int mode = 4;
  if (skip_unchanged && quad_changed[w] == 0) mode = 5;
  const wp::vec2 sums = sparse_newton_upstream_native(mat_of(H, @P@, w), row_of(grad, grad_ld, grad_ld, w),
                                                      mat_of(U, @P@, w), row_of(search, @NV@, @NV@, w), lane, mode);
  if (lane == 0) search_dot[w] = sums[0], decrement[w] = sums[1];
}
// ---- tree L'DL (@G@ groups) ----------------------------------------------------------------
__device__ void tree_ldl_native(fa M, fa y, fa x, int w, int nworld) {
@TREE@
}
__global__ void k_tree(fa M, fa y, fa x) { tree_ldl_native(M, y, x, blockIdx.x * blockDim.x + threadIdx.x, M.shape[0]); }
}  // namespace case_@NAME@
"""

LAUNCH = r"""
static int check(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { fprintf(stderr, "%s: %s\n", what, cudaGetErrorString(e)); return -1; }
  return 0;
}
extern "C" int ref_sparse_init(int c, const unsigned char* done, const int* nefc, const float* J, int njmax, const float* D,
                               const int* state, const float* M, int nM, const float* grad, int grad_ld, float* U,
                               float* search, float* search_dot, float* decrement, int nworld, void* stream) {
  switch (c) {
@INIT_CASES@
    default: return -2;
  }
  return check("ref_sparse_init");
}
extern "C" int ref_sparse_fused(int c, const float* J, int njmax, const float* D, const int* state, const int* ids,
                                const int* count, const int* uni, const float* grad, int grad_ld, float* U, float* search,
                                float* search_dot, float* decrement, int mode, int nworld, void* stream) {
  switch (c) {
@FUSED_CASES@
    default: return -2;
  }
  return check("ref_sparse_fused");
}
extern "C" int ref_sparse_nonfused(int c, const unsigned char* done, const float* grad, int grad_ld, const float* H,
                                   const int* quad_changed, const int* state_changed, float* U, float* search,
                                   float* search_dot, float* decrement, int skip_unchanged, int skip_noflip, int nworld,
                                   void* stream) {
  switch (c) {
@NONFUSED_CASES@
    default: return -2;
  }
  return check("ref_sparse_nonfused");
}
extern "C" int ref_tree_ldl(int c, const float* M, int nM, const float* y, float* x, int nworld, void* stream) {
  switch (c) {
@TREE_CASES@
    default: return -2;
  }
  return check("ref_tree_ldl");
}
"""


def _stand_ins() -> None:
    """``warp`` (its decorators are reached only inside factories this script never calls)
    and the reference's upstream shim, of which build_plan reads one enum value."""
    sys.modules.setdefault("warp", types.ModuleType("warp"))

    class ConstraintState(enum.IntEnum):
        QUADRATIC = 1

    chain = "instantmimic.utils.mjw_kernels.private".split(".")
    for k in range(1, len(chain) + 1):
        sys.modules.setdefault(".".join(chain[:k]), types.ModuleType(".".join(chain[:k])))
    sys.modules["instantmimic.utils.mjw_kernels.private"].types = types.SimpleNamespace(ConstraintState=ConstraintState)


def load(root: Path, name: str):
    _stand_ins()
    path = root / "src" / "instantmimic" / "utils" / "mjw_kernels" / f"{name}.py"
    spec = importlib.util.spec_from_file_location(f"ref_{name}", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


class _Arr:
    def __init__(self, a):
        self._a = np.asarray(a)
        self.shape, self.size = self._a.shape, self._a.size

    def numpy(self):
        return self._a


def adapt(m):
    out = types.SimpleNamespace(nv=m.nv, nv_pad=m.nv_pad, neq=0, nflex=0, ntendon=0)
    for name in ("dof_parentid", "body_parentid", "body_dofadr", "body_dofnum", "geom_bodyid", "nxn_geom_pair_filtered",
                 "M_colind", "M_hinit_i"):
        setattr(out, name, _Arr(getattr(m, name)))
    return out


def case_models():
    """(name, host Model, body groups): the bench workloads and one nv = 64 point, every
    body its own group (what the bench and the parity tests declare)."""
    from instantmimic_b200 import synthetic

    single = lambda m: [[b] for b in range(1, len(m.body_dofadr))]  # noqa: E731
    for name in ("humanoid", "snu", "g1"):
        m, _, _ = synthetic.make_workload(name, 1)
        yield name, m, single(m)
    m, _, _ = synthetic.make_sweep_point(64, 32, 1)
    yield "limbs64", m, single(m)
    # rows that couple two limbs (both feet, both hands with the head): the pattern gets
    # entries outside the tree's own (fill), the factor levels wider teams
    m, _, _ = synthetic.make_workload("humanoid", 1)
    leaves = leaf_bodies(m)
    yield "humanoid_pairs", m, [leaves[:2], leaves[2:]] + [[b] for b in range(1, len(m.body_dofadr)) if b not in leaves]


def leaf_bodies(m) -> list[int]:
    parents = set(np.asarray(m.body_parentid)[1:].tolist())
    return [b for b in range(1, len(m.body_dofadr)) if b not in parents]


def body_chain(m, body: int) -> list[int]:
    """Dofs of a body and of all its ancestors."""
    first, count = int(m.body_dofadr[body]), int(m.body_dofnum[body])
    dof, chain = first + count - 1, []
    while dof >= 0:
        chain.append(dof)
        dof = int(m.dof_parentid[dof])
    return sorted(chain)


def rows_for_groups(m, groups, nworld: int, njmax: int, rng) -> np.ndarray:
    """Constraint Jacobians whose rows stay inside the declared coupling: every row takes
    one or two bodies of one group and is nonzero on the dofs of their chains."""
    J = np.zeros((nworld, njmax, m.nv), np.float32)
    for w in range(nworld):
        for r in range(njmax):
            group = groups[int(rng.integers(len(groups)))]
            pick = rng.choice(group, size=min(len(group), int(rng.integers(1, 3))), replace=False)
            dofs = sorted({d for b in pick for d in body_chain(m, int(b))})
            J[w, r, dofs] = rng.normal(size=len(dofs))
    return J


def indent(text: str) -> str:
    return "\n".join("  " + line for line in text.splitlines())


def generate(root: Path) -> tuple[str, list[dict]]:
    sh, tl = load(root, "sparse_hessian"), load(root, "tree_ldl")
    parts, manifest = [SHIM], []
    sw = {k: [] for k in ("INIT", "FUSED", "NONFUSED", "TREE")}
    for index, (name, m, groups) in enumerate(case_models()):
        fb = 32 if m.nv_pad < 64 else 64
        fused = sh.build_plan(adapt(m), groups, fb, "fused")
        nonfused = sh.build_plan(adapt(m), groups, 64, "nonfused")
        st = tl.tree_ldl_structure(np.asarray(m.M_rowadr), np.asarray(m.M_rownnz), np.asarray(m.M_colind))
        plan = tl.best_tree_ldl_plan(*st)
        tree = tl._generate_source(*st, plan, True)
        g = len(plan.groups)
        text = CASE
        for key, val in (("@NAME@", name), ("@FB@", str(fb)), ("@NB@", "64"), ("@G@", str(g)), ("@P@", str(m.nv_pad)),
                         ("@NV@", str(m.nv)), ("@FACTOR@", indent(fused.factor_snippet)),
                         ("@INIT@", indent(fused.init_snippet)), ("@NONFUSED@", indent(nonfused.nonfused_snippet)),
                         ("@TREE@", indent(tree))):
            text = text.replace(key, val)
        parts.append(text)
        ns, P, nv = f"case_{name}", m.nv_pad, m.nv
        s = "(cudaStream_t)stream"
        sw["INIT"].append(
            f"    case {index}: {ns}::k_init<<<nworld, {fb}, 0, {s}>>>(done, nefc, make3(J, nworld, njmax, {nv}), "
            f"make2(D, nworld, njmax), make2(state, nworld, njmax), make2(M, nworld, nM), grad, grad_ld, U, search, "
            f"search_dot, decrement); break;")
        sw["FUSED"].append(
            f"    case {index}: {ns}::k_fused<<<nworld, {fb}, 0, {s}>>>(make3(J, nworld, njmax, {nv}), "
            f"make2(D, nworld, njmax), make2(state, nworld, njmax), make2(ids, nworld, njmax), count, "
            f"make2(uni, nworld, {nv + 1}), grad, grad_ld, U, search, search_dot, decrement, mode); break;")
        sw["NONFUSED"].append(
            f"    case {index}: {ns}::k_nonfused<<<nworld, 64, 0, {s}>>>(done, grad, grad_ld, H, quad_changed, "
            f"state_changed, U, search, search_dot, decrement, skip_unchanged, skip_noflip); break;")
        sw["TREE"].append(
            f"    case {index}: {ns}::k_tree<<<(nworld + 31) / 32, {32 * g}, 0, {s}>>>(make2(M, nworld, nM), "
            f"make2(y, nworld, {nv}), make2(x, nworld, {nv})); break;")
        manifest.append({"name": name, "index": index, "nv": nv, "nv_pad": P, "nM": int(m.nM), "fused_block": fb,
                         "nonfused_block": 64, "nfac_fused": int(fused.nslots - nv), "nfac_nonfused": int(nonfused.nslots - nv),
                         "tree_groups": g})
    launch = LAUNCH
    for key, lines in sw.items():
        launch = launch.replace(f"@{key}_CASES@", "\n".join(lines))
    parts.append(launch)
    return "\n".join(parts), manifest


def build(root: Path = Path("/root/reference"), verbose: bool = False) -> Path:
    """Generates and compiles; raises when the reference tree or nvcc is missing."""
    if not (root / "src" / "instantmimic" / "utils" / "mjw_kernels" / "sparse_hessian.py").exists():
        raise FileNotFoundError(f"no reference tree at {root}")
    from instantmimic_b200.build import nvcc

    OUT.mkdir(exist_ok=True)
    source, manifest = generate(root)
    cu = OUT / "ref_snippets.cu"
    cu.write_text(source)
    # nvcc's defaults on purpose: -fmad=true is how Warp compiles the same text
    cmd = [nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-shared",
           "-o", str(LIB), str(cu)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed on the reference snippets")
    MANIFEST.write_text(json.dumps(manifest, indent=1))
    return LIB


def manifest() -> list[dict]:
    return json.loads(MANIFEST.read_text())


if __name__ == "__main__":
    print(build(Path(sys.argv[1]) if len(sys.argv) > 1 else Path("/root/reference"), verbose=True))
