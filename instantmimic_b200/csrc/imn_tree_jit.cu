// imn_tree_jit.cu -- the tree L'DL plan as generated straight-line code.
//
// The reference turns a TreeLdlPlan into source text and compiles it at run time
// (tree_ldl.py:196-359 _generate_source, tree_ldl.py:362-390
// make_tree_ldl_factor_solve_kernel).  This file does the same for sm_100a: it writes
// CUDA C from the plan's instruction list, compiles it with NVRTC (loaded with dlopen,
// so the library itself does not depend on it) and launches the result through the
// runtime's library API.  The mapping is the plan's: a block serves 32 worlds with one
// warp per group, lane l works on world 32*block + l, the trunk runs on the owner
// warp between two block barriers.
//
// What the generator adds over interpreting the list (imn_tree_ldl_solve): a slot
// that only one warp ever touches becomes a register variable of that warp's
// straight-line code, so the elimination runs from registers with no instruction
// decode; only the values that cross warps (the groups' contributions to the trunk and
// the trunk's solution) go through shared memory, column = lane.  Every statement is
// the instruction's own float32 operation (explicit fmaf, IEEE division, contraction
// off), in list order, so the results are bit-identical to the interpreter's.
//
// Memory.  Lane = world means that a plain load of M[world][e] touches 32 cache lines
// per instruction, and the L1's one-line-per-cycle rate, not HBM, then bounds the
// kernel (nM such loads per 32 worlds).  The generated kernel therefore stages its
// block's tile -- 32 worlds x nM floats of M and 32 x nv of y, both contiguous -- in
// shared memory: two TMA bulk copies on one mbarrier when the tile is whole and
// 16-byte aligned (bounded wait), cooperative coalesced loads otherwise.  The
// straight-line code reads the tile (stride nM between lanes: gcd(nM, 32)-way bank
// conflicts), writes x over the consumed y, and the tile leaves by one bulk store.
// Plans whose tile does not fit twice into an SM's shared memory, or whose nM shares
// a factor of 8 or more with 32, keep the plain loads.
#include <dlfcn.h>
#include <stdlib.h>

#include <mutex>
#include <string>
#include <vector>

#include "imn_common.cuh"

namespace {

enum { OP_LOAD_M, OP_LOAD_Y, OP_ZERO, OP_INV, OP_UPD, OP_SCALE, OP_SUBMUL, OP_MUL, OP_ADD, OP_STORE_X, OP_MULSUB, OP_MULADD };

// ---- NVRTC through dlopen ---------------------------------------------------------
typedef void* nvrtcProgram_t;
struct Nvrtc {
  void* handle = nullptr;
  int (*create)(nvrtcProgram_t*, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
  int (*compile)(nvrtcProgram_t, int, const char* const*) = nullptr;
  int (*log_size)(nvrtcProgram_t, size_t*) = nullptr;
  int (*log)(nvrtcProgram_t, char*) = nullptr;
  int (*cubin_size)(nvrtcProgram_t, size_t*) = nullptr;
  int (*cubin)(nvrtcProgram_t, char*) = nullptr;
  int (*destroy)(nvrtcProgram_t*) = nullptr;
  const char* (*error_string)(int) = nullptr;
};

bool nvrtc_open(Nvrtc& api);

Nvrtc* nvrtc() {
  static Nvrtc api;
  static std::once_flag once;
  std::call_once(once, [] { nvrtc_open(api); });
  return api.handle ? &api : nullptr;
}

bool nvrtc_open(Nvrtc& api) {
  const char* names[] = {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12",
                         "/usr/local/cuda/lib64/libnvrtc.so"};
  void* h = nullptr;
  for (const char* n : names)
    if ((h = dlopen(n, RTLD_NOW | RTLD_LOCAL))) break;
  if (!h) return false;
#define IMN_SYM(field, name)                                        \
  api.field = reinterpret_cast<decltype(api.field)>(dlsym(h, name)); \
  if (!api.field) return false
  IMN_SYM(create, "nvrtcCreateProgram");
  IMN_SYM(compile, "nvrtcCompileProgram");
  IMN_SYM(log_size, "nvrtcGetProgramLogSize");
  IMN_SYM(log, "nvrtcGetProgramLog");
  IMN_SYM(cubin_size, "nvrtcGetCUBINSize");
  IMN_SYM(cubin, "nvrtcGetCUBIN");
  IMN_SYM(destroy, "nvrtcDestroyProgram");
  IMN_SYM(error_string, "nvrtcGetErrorString");
#undef IMN_SYM
  api.handle = h;
  return true;
}

struct Ins {
  int op, dst, a, b, c;
};

// operands an instruction reads / the slot it writes (-1: none)
void operands(const Ins& i, int reads[4], int& nread, int& write) {
  nread = 0, write = -1;
  switch (i.op) {
    case OP_LOAD_M:
    case OP_LOAD_Y:
    case OP_ZERO: write = i.dst; break;
    case OP_INV: reads[nread++] = i.a, write = i.dst; break;
    case OP_UPD: reads[nread++] = i.a, reads[nread++] = i.b, reads[nread++] = i.c, reads[nread++] = i.dst, write = i.dst; break;
    case OP_SCALE: reads[nread++] = i.a, reads[nread++] = i.dst, write = i.dst; break;
    case OP_SUBMUL: reads[nread++] = i.a, reads[nread++] = i.b, reads[nread++] = i.dst, write = i.dst; break;
    case OP_MUL: reads[nread++] = i.a, reads[nread++] = i.b, write = i.dst; break;
    case OP_ADD: reads[nread++] = i.a, reads[nread++] = i.dst, write = i.dst; break;
    case OP_MULSUB:
    case OP_MULADD: reads[nread++] = i.a, reads[nread++] = i.b, reads[nread++] = i.dst, write = i.dst; break;
    case OP_STORE_X: reads[nread++] = i.a; break;
    default: break;
  }
}

}  // namespace

struct ImnTreeKernel {
  int nv = 0, nM = 0, groups = 0;
  int nshared = 0;   // values that cross warps
  int nexchange = 0;  // of those, the ones that need shared memory of their own
  int min_blocks = 1;  // register bound of the generated kernel
  bool staged = false;  // M and y tiles in shared memory
  std::string name;     // entry point of the generated source
  std::string source;
  std::vector<char> cubin;
  cudaLibrary_t library = nullptr;
  cudaKernel_t kernel = nullptr;
  std::mutex load_mutex;  // the first solve loads the machine code
};

namespace {

std::string generate(const std::string& name, const int32_t* prog, const int32_t* ptr, int groups, int owner,
                     int nslot, int nv, int nM, bool allow_stage, int min_blocks, bool* staged_out, int* nshared_out,
                     int* nexchange_out) {
  const int nstream = 2 * groups + 1;
  auto warp_of = [&](int st) { return st < groups ? st : (st == groups ? owner : st - groups - 1); };
  std::vector<std::vector<Ins>> streams(nstream);
  std::vector<unsigned> users(nslot, 0u);
  for (int st = 0; st < nstream; ++st)
    for (int pc = ptr[st]; pc < ptr[st + 1]; ++pc) {
      const int32_t* w = prog + 4 * pc;
      Ins i{w[0], w[1], w[2] & 0xFFFF, (w[2] >> 16) & 0xFFFF, w[3]};
      streams[st].push_back(i);
      int reads[4], nread, write;
      operands(i, reads, nread, write);
      for (int k = 0; k < nread; ++k) users[reads[k]] |= 1u << warp_of(st);
      if (write >= 0) users[write] |= 1u << warp_of(st);
    }
  // slots that more than one warp touches live in shared memory
  std::vector<int> shared_index(nslot, -1);
  int nshared = 0;
  for (int sl = 0; sl < nslot; ++sl)
    if (users[sl] & (users[sl] - 1u)) shared_index[sl] = nshared++;
  *nshared_out = nshared;
  // A staged tile has room for most of the exchange: once a warp has read an entry of M
  // into a register, nobody reads that cell of the tile again (an entry is loaded once),
  // so a cross-warp value first written by the same warp later on can live there.  Cells
  // are handed out in program order, phase by phase; within a phase a cross-warp value is
  // touched by one warp only (the exchange goes through the block barriers), so the first
  // touch found here is the first in time.  Values that find no cell keep a slot of their own.
  std::vector<int> cell(nslot, -1);
  int nexchange = nshared;
  const size_t tile_only = 16 + sizeof(float) * ((size_t)((32 * nM + 3) & ~3) + ((32 * nv + 3) & ~3));
  if (allow_stage && tile_only + 128 <= 113 * 1024) {
    std::vector<int> loads(nM, 0);
    for (const auto& code : streams)
      for (const Ins& i : code)
        if (i.op == OP_LOAD_M) ++loads[i.a];
    std::vector<std::vector<int>> freed(groups);
    std::vector<char> seen(nslot, 0);
    for (int st = 0; st < nstream; ++st) {
      const int w = warp_of(st);
      for (const Ins& i : streams[st]) {
        int reads[4], nread, write;
        operands(i, reads, nread, write);
        for (int k = 0; k < nread; ++k) seen[reads[k]] = 1;
        if (write >= 0 && shared_index[write] >= 0 && !seen[write] && !freed[w].empty()) {
          cell[write] = freed[w].back();
          freed[w].pop_back();
        }
        if (write >= 0) seen[write] = 1;
        if (i.op == OP_LOAD_M && loads[i.a] == 1) freed[w].push_back(i.a);
      }
    }
    // the values left over are renumbered densely
    nexchange = 0;
    for (int sl = 0; sl < nslot; ++sl)
      if (shared_index[sl] >= 0 && cell[sl] < 0) shared_index[sl] = nexchange++;
  }
  *nexchange_out = nexchange;
  // stage the tiles when two blocks' worth fit an SM's shared memory
  const size_t tile_bytes = tile_only + sizeof(float) * 32 * (size_t)(nexchange > 0 ? nexchange : 1);
  const bool staged = allow_stage && tile_bytes <= 113 * 1024;
  *staged_out = staged;
  if (!staged && nexchange != nshared) {
    // plain loads: no tile to lend cells, every cross-warp value has its own slot
    nexchange = 0;
    for (int sl = 0; sl < nslot; ++sl)
      if (shared_index[sl] >= 0) cell[sl] = -1, shared_index[sl] = nexchange++;
    *nexchange_out = nexchange;
  }
  auto ref = [&](int sl) {
    if (shared_index[sl] < 0) return "r" + std::to_string(sl);
    if (cell[sl] >= 0) return "Mw[" + std::to_string(cell[sl]) + "]";
    return "S[" + std::to_string(shared_index[sl] * 32) + "]";
  };
  auto emit = [&](std::string& out, const std::vector<Ins>& code) {
    for (const Ins& i : code) {
      const std::string d = i.op == OP_STORE_X ? "" : ref(i.dst);
      switch (i.op) {
        case OP_LOAD_M: out += d + (staged ? " = Mt[" : " = Mr[") + std::to_string(i.a) + "];\n"; break;
        case OP_LOAD_Y: out += d + (staged ? " = yt[" : " = yr[") + std::to_string(i.a) + "];\n"; break;
        case OP_ZERO: out += d + " = 0.0f;\n"; break;
        case OP_INV: out += d + " = 1.0f / " + ref(i.a) + ";\n"; break;
        case OP_UPD:
          out += d + " = fmaf(-(" + ref(i.a) + " * " + ref(i.b) + "), " + ref(i.c) + ", " + d + ");\n";
          break;
        case OP_SCALE: out += d + " = " + d + " * " + ref(i.a) + ";\n"; break;
        case OP_SUBMUL: out += d + " = fmaf(-" + ref(i.a) + ", " + ref(i.b) + ", " + d + ");\n"; break;
        case OP_MUL: out += d + " = " + ref(i.a) + " * " + ref(i.b) + ";\n"; break;
        case OP_ADD: out += d + " = " + d + " + " + ref(i.a) + ";\n"; break;
        case OP_MULSUB: out += d + " = fmaf(" + ref(i.a) + ", " + ref(i.b) + ", -" + d + ");\n"; break;
        case OP_MULADD: out += d + " = fmaf(" + ref(i.a) + ", " + ref(i.b) + ", " + d + ");\n"; break;
        case OP_STORE_X:
          out += staged ? "yt[" + std::to_string(i.dst) + "] = " + ref(i.a) + ";\n"
                        : "if (live) xr[" + std::to_string(i.dst) + "] = " + ref(i.a) + ";\n";
          break;
        default: break;
      }
    }
  };
  std::string src;
  const std::string threads = std::to_string(32 * groups);
  src += "extern \"C\" __global__ void __launch_bounds__(" + threads + ", " + std::to_string(min_blocks) +
         ") " + name + "(const float* __restrict__ M, long long M_ld, const float* __restrict__ y,\n"
         "    long long y_ld, float* __restrict__ x, long long x_ld, int nworld, int bulk) {\n"
         "  extern __shared__ __align__(16) float slots[];\n"
         "  const int lw = threadIdx.x & 31, part = threadIdx.x >> 5;\n"
         "  const int world = blockIdx.x * 32 + lw;\n"
         "  const bool live = world < nworld;\n"
         "  const int src = live ? world : nworld - 1;\n";
  if (!staged) {
    src += "  const float* Mr = M + (long long)src * M_ld;\n"
           "  const float* yr = y + (long long)src * y_ld;\n"
           "  float* xr = x + (long long)src * x_ld;\n"
           "  float* S = slots + lw;\n";
  } else {
    // tile layout: [bar 16 B][M 32 x nM][y 32 x nv][cross-warp slots]
    const int nMt = 32 * nM, nyt = 32 * nv;
    const std::string sM = std::to_string(nM), sV = std::to_string(nv);
    src += "  float* tileM = slots + 4;\n"
           "  float* tileY = tileM + " + std::to_string((nMt + 3) & ~3) + ";\n"
           "  float* S = tileY + " + std::to_string((nyt + 3) & ~3) + " + lw;\n"
           "  const float* Mt = tileM + lw * " + sM + ";\n"
           "  float* Mw = tileM + lw * " + sM + ";  // cells of entries already read hold exchanged values\n"
           "  float* yt = tileY + lw * " + sV + ";\n"
           "  const int w0 = blockIdx.x * 32;\n"
           "  const bool whole = bulk && w0 + 32 <= nworld;\n"
           "  const unsigned bar = (unsigned)__cvta_generic_to_shared(slots);\n"
           "  bool arrived = false;\n"
           "  if (whole) {\n"
           "    if (threadIdx.x == 0) {\n"
           "      asm volatile(\"mbarrier.init.shared::cta.b64 [%0], 1;\" ::\"r\"(bar) : \"memory\");\n"
           "      asm volatile(\"fence.mbarrier_init.release.cluster;\" ::: \"memory\");\n"
           "      asm volatile(\"mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\" ::\"r\"(bar), \"r\"(" +
           std::to_string(4 * (nMt + nyt)) + "u) : \"memory\");\n"
           "      asm volatile(\"cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\"\n"
           "                   ::\"r\"((unsigned)__cvta_generic_to_shared(tileM)), \"l\"(M + (long long)w0 * " + sM + "), \"r\"(" +
           std::to_string(4 * nMt) + "u), \"r\"(bar) : \"memory\");\n"
           "      asm volatile(\"cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\"\n"
           "                   ::\"r\"((unsigned)__cvta_generic_to_shared(tileY)), \"l\"(y + (long long)w0 * " + sV + "), \"r\"(" +
           std::to_string(4 * nyt) + "u), \"r\"(bar) : \"memory\");\n"
           "    }\n"
           "    __syncthreads();  // the barrier is initialised before anyone polls it\n"
           "    // bounded wait; when it runs out the copies get one more bounded wait and the\n"
           "    // tile is then loaded again with plain loads\n"
           "    for (int round = 0; round < 2 && !arrived; ++round)\n"
           "      for (int tries = 0; tries < (1 << 22) && !arrived; ++tries) {\n"
           "        unsigned ok;\n"
           "        asm volatile(\"{\\n\\t.reg .pred p;\\n\\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\\n\\tselp.u32 %0, 1, 0, p;\\n\\t}\"\n"
           "                     : \"=r\"(ok) : \"r\"(bar) : \"memory\");\n"
           "        arrived = ok != 0;\n"
           "      }\n"
           "  }\n"
           "  if (!__syncthreads_and(arrived)) {\n"
           "    // partial or unaligned tile (or a copy that did not arrive): coalesced loads;\n"
           "    // lanes past the last world repeat it\n"
           "    for (int e = threadIdx.x; e < " + std::to_string(nMt) + "; e += " + threads + ") {\n"
           "      const int r = e / " + sM + ", c = e - r * " + sM + ";\n"
           "      const int wr = w0 + r < nworld ? w0 + r : nworld - 1;\n"
           "      tileM[e] = M[(long long)wr * M_ld + c];\n"
           "    }\n"
           "    for (int e = threadIdx.x; e < " + std::to_string(nyt) + "; e += " + threads + ") {\n"
           "      const int r = e / " + sV + ", c = e - r * " + sV + ";\n"
           "      const int wr = w0 + r < nworld ? w0 + r : nworld - 1;\n"
           "      tileY[e] = y[(long long)wr * y_ld + c];\n"
           "    }\n"
           "    __syncthreads();\n"
           "  }\n";
  }
  src += "  switch (part) {\n";
  for (int j = 0; j < groups; ++j) {
    src += "  case " + std::to_string(j) + ": {\n";
    // register variables of this warp
    int n = 0;
    for (int sl = 0; sl < nslot; ++sl)
      if (shared_index[sl] < 0 && users[sl] == (1u << j)) {
        src += (n % 8 == 0 ? std::string(n ? ";\nfloat " : "float ") : std::string(", ")) + "r" + std::to_string(sl) +
               " = 0.0f";
        ++n;
      }
    if (n) src += ";\n";
    emit(src, streams[j]);
    src += "asm volatile(\"bar.sync 0;\" ::: \"memory\");\n";
    if (j == owner) emit(src, streams[groups]);
    src += "asm volatile(\"bar.sync 0;\" ::: \"memory\");\n";
    emit(src, streams[groups + 1 + j]);
    src += "  } break;\n";
  }
  src += "  default: break;\n  }\n";
  if (staged) {
    const std::string sV = std::to_string(nv);
    src += "  // every thread's writes of x become visible to the bulk store's proxy\n"
           "  asm volatile(\"fence.proxy.async.shared::cta;\" ::: \"memory\");\n"
           "  __syncthreads();  // x of every world is in the tile\n"
           "  if (whole && x_ld == " + sV + ") {\n"
           "    if (threadIdx.x == 0) {\n"
           "      asm volatile(\"cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\"\n"
           "                   ::\"l\"(x + (long long)w0 * " + sV + "), \"r\"((unsigned)__cvta_generic_to_shared(tileY)), \"r\"(" +
           std::to_string(4 * 32 * nv) + "u) : \"memory\");\n"
           "      asm volatile(\"cp.async.bulk.commit_group;\" ::: \"memory\");\n"
           "      asm volatile(\"cp.async.bulk.wait_group.read 0;\" ::: \"memory\");\n"
           "    }\n"
           "  } else {\n"
           "    for (int e = threadIdx.x; e < " + std::to_string(32 * nv) + "; e += " + threads + ") {\n"
           "      const int r = e / " + sV + ", c = e - r * " + sV + ";\n"
           "      if (w0 + r < nworld) x[(long long)(w0 + r) * x_ld + c] = tileY[e];\n"
           "    }\n"
           "  }\n";
  }
  src += "}\n";
  return src;
}

}  // namespace

// Checks a program, writes its source and compiles it; `what` names the caller in errors.
static int compile_program(const char* what, const char* name, const int32_t* prog, const int32_t* prog_ptr, int32_t nv,
                           int32_t nM, int32_t groups, int32_t owner, int32_t nslot, int min_blocks,
                           ImnTreeKernel** out) {
  if (!prog || !prog_ptr || !out) return imn::set_error("%s: NULL argument", what), IMN_ERR_NULL;
  *out = nullptr;
  if (nv <= 0 || groups < 1 || groups > 4 || owner < 0 || owner >= groups || nslot <= 0 || nslot > (1 << 16))
    return imn::set_error("%s: malformed plan", what), IMN_ERR_SHAPE;
  const int nstream = 2 * groups + 1;
  for (int st = 0; st < nstream; ++st)
    if (prog_ptr[st] > prog_ptr[st + 1] || prog_ptr[st] < 0)
      return imn::set_error("%s: stream offsets are not ascending", what), IMN_ERR_SHAPE;
  for (int pc = 0; pc < prog_ptr[nstream]; ++pc) {
    const int32_t* w = prog + 4 * pc;
    const int dst = w[1], a = w[2] & 0xFFFF, b = (w[2] >> 16) & 0xFFFF, c = w[3];
    const bool index_a = w[0] == OP_LOAD_M || w[0] == OP_LOAD_Y;  // a addresses M or y
    const bool index_d = w[0] == OP_STORE_X;                      // dst addresses x
    if (w[0] < 0 || w[0] > OP_MULADD || dst < 0 || (!index_d && dst >= nslot) || (index_d && dst >= nv) ||
        (!index_a && a >= nslot) || (w[0] == OP_LOAD_M && a >= nM) || (w[0] == OP_LOAD_Y && a >= nv) || b >= nslot ||
        c < 0 || c >= nslot)
      return imn::set_error("%s: instruction %d is out of range", what, pc), IMN_ERR_SHAPE;
  }
  Nvrtc* rt = nvrtc();
  if (!rt) return imn::set_error("%s: NVRTC (libnvrtc.so.12) could not be loaded", what), IMN_ERR_UNSUPPORTED;
  ImnTreeKernel* k = new ImnTreeKernel;
  k->nv = nv, k->nM = nM, k->groups = groups, k->name = name;
  {
    // stage when two blocks' tiles fit an SM and the lane stride nM does not pile the
    // lanes onto a few banks; IMN_TREE_STAGE=0 keeps the plain loads (for comparisons)
    int gcd = nM, b = 32;
    while (b) {
      const int t = gcd % b;
      gcd = b, b = t;
    }
    const char* env = getenv("IMN_TREE_STAGE");
    k->staged = !(env && env[0] == '0') && gcd < 8;
  }
  // The register bound follows from the shared memory the kernel will ask for: a first
  // pass of the generator sizes the exchange, the second writes the source with
  // __launch_bounds__(threads, blocks an SM's shared memory holds, at most `min_blocks`).
  // IMN_TREE_MIN_BLOCKS overrides the bound (for comparisons).
  generate(k->name, prog, prog_ptr, groups, owner, nslot, nv, nM, k->staged, 1, &k->staged, &k->nshared, &k->nexchange);
  {
    size_t bytes = (size_t)(k->nexchange > 0 ? k->nexchange : 1) * 32 * sizeof(float);
    if (k->staged) bytes += 16 + sizeof(float) * ((size_t)((32 * nM + 3) & ~3) + ((32 * nv + 3) & ~3));
    const int fit = (int)((228 * 1024) / (bytes + 1024));
    const char* env = getenv("IMN_TREE_MIN_BLOCKS");
    k->min_blocks = env && atoi(env) > 0 ? atoi(env) : (fit < 1 ? 1 : (fit > min_blocks ? min_blocks : fit));
  }
  k->source = generate(k->name, prog, prog_ptr, groups, owner, nslot, nv, nM, k->staged, k->min_blocks, &k->staged,
                       &k->nshared, &k->nexchange);
  nvrtcProgram_t p = nullptr;
  int rc = rt->create(&p, k->source.c_str(), (k->name + ".cu").c_str(), 0, nullptr, nullptr);
  if (rc) {
    imn::set_error("%s: nvrtcCreateProgram: %s", what, rt->error_string(rc));
    delete k;
    return IMN_ERR_LAUNCH;
  }
  const char* opts[] = {"--gpu-architecture=sm_100a", "--fmad=false", "--std=c++17", "-lineinfo"};
  rc = rt->compile(p, 4, opts);
  if (rc) {
    size_t n = 0;
    rt->log_size(p, &n);
    std::string log(n, '\0');
    if (n) rt->log(p, &log[0]);
    imn::set_error("%s: %s: %.380s", what, rt->error_string(rc), log.c_str());
    rt->destroy(&p);
    delete k;
    return IMN_ERR_LAUNCH;
  }
  size_t n = 0;
  rt->cubin_size(p, &n);
  k->cubin.resize(n);
  if (n) rt->cubin(p, k->cubin.data());
  rt->destroy(&p);
  if (!n) {
    imn::set_error("%s: NVRTC produced no machine code", what);
    delete k;
    return IMN_ERR_LAUNCH;
  }
  *out = k;
  return IMN_OK;
}

extern "C" int imn_tree_ldl_compile(const int32_t* prog, const int32_t* prog_ptr, int32_t nv, int32_t nM,
                                    int32_t groups, int32_t owner, int32_t nslot, ImnTreeKernel** out) {
  return compile_program("imn_tree_ldl_compile", "tree_ldl_generated", prog, prog_ptr, nv, nM, groups, owner, nslot, 4,
                         out);
}

// out = M v as a program of the same kind: before the first block barrier every warp
// loads the entries of v its rows need into registers, after the second it forms its
// rows' sums in the order of the symmetric-row table (one fmaf per stored entry, M read
// once from the staged tile, no table and no v reads at run time) and stores them over
// the tile of v, which leaves by the bulk store.
extern "C" int imn_mul_m_compile(const int32_t* prog, const int32_t* prog_ptr, int32_t nv, int32_t nM, int32_t groups,
                                 int32_t nslot, ImnTreeKernel** out) {
  return compile_program("imn_mul_m_compile", "mul_m_generated", prog, prog_ptr, nv, nM, groups, 0, nslot, 6, out);
}

extern "C" int imn_tree_ldl_kernel_info(const ImnTreeKernel* k, int32_t* shared_slots, int64_t* code_bytes,
                                        const char** source) {
  if (!k) return imn::set_error("imn_tree_ldl_kernel_info: NULL kernel"), IMN_ERR_NULL;
  if (shared_slots) *shared_slots = k->nshared;
  if (code_bytes) *code_bytes = (int64_t)k->cubin.size();
  if (source) *source = k->source.c_str();
  return IMN_OK;
}

extern "C" void imn_tree_ldl_kernel_destroy(ImnTreeKernel* k) {
  if (!k) return;
  if (k->library) cudaLibraryUnload(k->library);
  delete k;
}

extern "C" int imn_tree_ldl_compiled_solve(ImnTreeKernel* k, const float* M, int64_t M_ld, const float* y,
                                           int64_t y_ld, float* x, int64_t x_ld, int32_t nworld, void* stream) {
  if (!k || !M || !y || !x) return imn::set_error("imn_tree_ldl_compiled_solve: NULL argument"), IMN_ERR_NULL;
  if (nworld < 0 || M_ld < k->nM || y_ld < k->nv || x_ld < k->nv)
    return imn::set_error("imn_tree_ldl_compiled_solve: a stride is smaller than its extent"), IMN_ERR_SHAPE;
  if (nworld == 0) return IMN_OK;
  size_t bytes = (size_t)(k->nexchange > 0 ? k->nexchange : 1) * 32 * sizeof(float);
  if (k->staged) bytes += 16 + sizeof(float) * ((size_t)((32 * k->nM + 3) & ~3) + ((32 * k->nv + 3) & ~3));
  if (bytes > 227 * 1024)
    return imn::set_error("imn_tree_ldl_compiled_solve: %zu bytes of shared memory per block (max %d)", bytes,
                          227 * 1024),
           IMN_ERR_LIMIT;
  std::unique_lock<std::mutex> lock(k->load_mutex);
  if (!k->kernel) {
    // first use: hand the machine code to the runtime (do this outside stream capture)
    cudaError_t e = cudaLibraryLoadData(&k->library, k->cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
    if (e == cudaSuccess) e = cudaLibraryGetKernel(&k->kernel, k->library, k->name.c_str());
    if (e == cudaSuccess && bytes > 48 * 1024)
      e = cudaFuncSetAttribute(reinterpret_cast<const void*>(k->kernel), cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)bytes);
    if (e != cudaSuccess) {
      k->kernel = nullptr;
      return imn::set_error("imn_tree_ldl_compiled_solve: loading the generated kernel: %s", cudaGetErrorString(e)),
             IMN_ERR_LAUNCH;
    }
  }
  lock.unlock();
  long long mld = M_ld, yld = y_ld, xld = x_ld;
  int nw = nworld;
  // bulk copies need contiguous worlds and 16-byte aligned tiles (a tile is 32 worlds:
  // 128 nM and 128 nv bytes, so the base addresses decide)
  int bulk = k->staged && M_ld == k->nM && y_ld == k->nv && (reinterpret_cast<uintptr_t>(M) & 15) == 0 &&
             (reinterpret_cast<uintptr_t>(y) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  void* args[] = {&M, &mld, &y, &yld, &x, &xld, &nw, &bulk};
  cudaError_t e = cudaLaunchKernel(reinterpret_cast<const void*>(k->kernel), dim3((nworld + 31) / 32),
                                   dim3(32 * k->groups), args, bytes, (cudaStream_t)stream);
  if (e != cudaSuccess)
    return imn::set_error("imn_tree_ldl_compiled_solve: launch failed: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  return IMN_OK;
}
