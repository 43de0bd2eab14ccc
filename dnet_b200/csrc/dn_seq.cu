// dn_seq.cu -- C ABI of libdnet_b200_seq.so (include/dnet_b200_seq.h): host bookkeeping of the batched step --
// bound weight pointers, the page pool and the state slots, the staging of a step's batch description, and the
// launch sequence of a layer.  All arithmetic is in dn_seq_kernels.cuh.
#include "dn_seq_kernels.cuh"
#include "dn_gemm_tc.cuh"      // the tcgen05 / TMA GEMM the llama-family prefill runs on (namespace dn)
#include "../../include/dnet_b200_seq.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <new>
#include <type_traits>
#include <vector>

using namespace dnseq;

#define DN_OK 0
#define DN_EINVAL (-22)
#define DN_ENOMEM (-12)
#define DN_ENOENT (-2)
#define DN_ECUDA (-5)
#define DN_ENOSPC (-28)

static thread_local char g_err[512] = "";
static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
#define CK(...)                                                                                                 \
  do {                                                                                                          \
    cudaError_t e_ = (__VA_ARGS__);                                                                             \
    if (e_ != cudaSuccess)                                                                                      \
      return fail(DN_ECUDA, "%s failed: %s (%s:%d)", #__VA_ARGS__, cudaGetErrorString(e_), __FILE__, __LINE__); \
  } while (0)

static std::atomic<long long> g_launches{0};
static int g_device = -1;
static int g_sms = 0;
static size_t g_max_smem = 0;

// weight matrices and the activation buffers they multiply get TMA descriptors in bf16 mode
struct XMaps {
  CUtensorMap m[3];     // token tiles of 32 / 64 / 128 rows
  bool ok = false;
};
struct SeqLayer {
  dn_seq_layer_cfg c;
  const void* w[DN_SQ_COUNT];
  CUtensorMap tm[DN_SQ_COUNT];
  bool tm_ok[DN_SQ_COUNT];
  XMaps x_mo, x_act;            // the mixer's output buffer [MB, Co] and the feed-forward's [MB, ff]
  int Cq, Ck, Cv, Co;           // projection widths: q, k, v and the mixer's output before W_o
  int kv_index;                 // attention: which page pool (own or the one it borrows); -1 for delta
  size_t conv_off, delta_off;   // element offsets into a slot's carried conv inputs / fp32 delta state
  float* inv_freq;              // [rot/2] device
};

struct dn_seq_model {
  dn_seq_cfg cfg;
  std::vector<SeqLayer> L;
  const void *embed = nullptr, *final_norm = nullptr, *head = nullptr;
  size_t esz = 2;
  int S1 = 1, MB = 0, max_pages = 0;
  // scratch
  float *xs = nullptr, *y = nullptr, *pa = nullptr, *pb = nullptr, *qn = nullptr, *kn = nullptr, *vv = nullptr, *od = nullptr,
        *beta = nullptr, *decay = nullptr;
  void *h = nullptr, *uq = nullptr, *uk = nullptr, *uv = nullptr, *qb = nullptr, *mo = nullptr, *gt = nullptr, *act = nullptr;
  // state
  std::vector<void*> kpool, vpool;
  void* conv_state = nullptr;
  size_t conv_stride = 0;       // elements per slot
  float* delta_state = nullptr;
  size_t delta_stride = 0;
  std::vector<int> free_pages, free_slots;
  std::vector<std::vector<int>> pages;   // per slot
  std::vector<int> length;               // per slot, -1: closed
  XMaps x_h;                    // the normed activations [MB, W]
  CUtensorMap tm_head;
  bool tm_head_ok = false;
  unsigned int* tc_err = nullptr;   // set by a bounded in-kernel wait of the tcgen05 GEMM that ran out
  // decode steps (every entry brings one token) replay a captured graph per (entries, wanted rows): all kernel
  // arguments of such a step are fixed buffers, the batch description is read from the staging area
  bool graphs_on = true;
  std::map<std::pair<int, int>, std::pair<cudaGraphExec_t, long long>> graphs;   // -> (exec, kernels per replay)
  float* lg_buf = nullptr;          // [8][vocab] logits of a replayed step, copied to the caller's buffer
  // phase profiler (off by default): one event at every phase boundary of a step, read back by dn_seq_profile_read
  bool prof_on = false;
  std::vector<cudaEvent_t> prof_pool;
  std::vector<std::pair<int, cudaEvent_t>> prof_marks;
  double prof_ms[DN_SEQ_PH_COUNT] = {0};
  // staging
  int32_t *stage_h = nullptr, *stage_d = nullptr, *bt_h = nullptr, *bt_d = nullptr;
  size_t stage_ints = 0;
  cudaEvent_t staged = nullptr;
};

template <typename... KArgs, typename... Args>
static cudaError_t launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  g_launches++;
  kern<<<grid, block, smem, s>>>(static_cast<KArgs>(args)...);
  return cudaGetLastError();
}

extern "C" const char* dn_seq_last_error(void) { return g_err; }
extern "C" int64_t dn_seq_launch_count(void) { return (int64_t)g_launches.load(); }

extern "C" int dn_seq_init(int device) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    return fail(DN_ECUDA, "no CUDA device visible (%s): libdnet_b200_seq has no CPU fallback", cudaGetErrorString(e));
  if (device < 0 || device >= n) return fail(DN_EINVAL, "device %d out of range [0,%d)", device, n);
  CK(cudaSetDevice(device));
  cudaDeviceProp p;
  CK(cudaGetDeviceProperties(&p, device));
  if (p.major != 10) return fail(DN_EINVAL, "device %d is sm_%d%d; this library is built for sm_100a only", device, p.major, p.minor);
  g_sms = p.multiProcessorCount;
  g_max_smem = p.sharedMemPerBlockOptin;
  g_device = device;
  return DN_OK;
}

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static PFN_encodeTiled g_encode = nullptr;
// [rows, cols] bf16 row-major, box box_rows x 64 columns (one 128-byte swizzle span); false when the tensor cannot
// have one (pitch or base not a multiple of 16 bytes) -- such products run on the CUDA-core kernels
static bool make_tmap(CUtensorMap* out, const void* base, int rows, int cols, int box_rows) {
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
      return false;
    g_encode = (PFN_encodeTiled)fn;
  }
  if (!base || cols % 64 || ((uintptr_t)base & 15)) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return g_encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
static void make_xmaps(XMaps* x, const void* base, int rows, int cols) {
  x->ok = true;
  const int br[3] = {32, 64, 128};
  for (int i = 0; i < 3; i++) x->ok = x->ok && make_tmap(&x->m[i], base, rows, cols, br[i]);
}

template <class P>
static int dalloc(P** p, size_t bytes) {
  void* q = nullptr;
  if (cudaMalloc(&q, bytes ? bytes : 16) != cudaSuccess) return fail(DN_ENOMEM, "cudaMalloc of %zu bytes failed", bytes);
  *p = (P*)q;
  return DN_OK;
}

extern "C" int dn_seq_model_destroy(dn_seq_model* m) {
  if (!m) return DN_OK;
  cudaDeviceSynchronize();
  void* ptrs[] = {m->xs, m->y, m->pa, m->pb, m->qn, m->kn, m->vv, m->od, m->beta, m->decay, m->h, m->uq, m->uk, m->uv, m->qb,
                  m->mo, m->gt, m->act, m->conv_state, m->delta_state, m->stage_d, m->bt_d, m->tc_err};
  for (void* p : ptrs) if (p) cudaFree(p);
  for (auto& g : m->graphs) cudaGraphExecDestroy(g.second.first);
  if (m->lg_buf) cudaFree(m->lg_buf);
  for (auto& pm : m->prof_marks) cudaEventDestroy(pm.second);
  for (cudaEvent_t ev : m->prof_pool) cudaEventDestroy(ev);
  for (void* p : m->kpool) if (p) cudaFree(p);
  for (void* p : m->vpool) if (p) cudaFree(p);
  for (auto& l : m->L) if (l.inv_freq) cudaFree(l.inv_freq);
  if (m->stage_h) cudaFreeHost(m->stage_h);
  if (m->bt_h) cudaFreeHost(m->bt_h);
  if (m->staged) cudaEventDestroy(m->staged);
  delete m;
  return DN_OK;
}

extern "C" int dn_seq_model_create(const dn_seq_cfg* cfg, const dn_seq_layer_cfg* layers, dn_seq_model** out) {
  if (!cfg || !layers || !out) return fail(DN_EINVAL, "null argument");
  if (g_device < 0) return fail(DN_EINVAL, "dn_seq_init() has not been called");
  if (cfg->width <= 0 || cfg->vocab <= 0 || cfg->n_layers <= 0) return fail(DN_EINVAL, "width / vocab / n_layers must be positive");
  if (cfg->streams < 0 || cfg->streams > MAX_STREAMS) return fail(DN_EINVAL, "streams %d unsupported (0..%d)", cfg->streams, MAX_STREAMS);
  if (cfg->dtype != DN_SEQ_BF16 && cfg->dtype != DN_SEQ_F32) return fail(DN_EINVAL, "dtype %d unsupported", cfg->dtype);
  if (cfg->pool_pages <= 0 || cfg->max_seqs <= 0 || cfg->max_batch_tokens <= 0) return fail(DN_EINVAL, "pool / slots / batch must be positive");
  dn_seq_model* m = new (std::nothrow) dn_seq_model();
  if (!m) return fail(DN_ENOMEM, "out of host memory");
  m->cfg = *cfg;
  m->esz = cfg->dtype == DN_SEQ_F32 ? 4 : 2;
  m->S1 = cfg->streams > 0 ? cfg->streams : 1;
  m->MB = cfg->max_batch_tokens;
  m->max_pages = cfg->pool_pages;
  m->L.resize(cfg->n_layers);
  int mq = 1, mk = 1, mv = 1, mo = 1, mh = 1, mff = 1, mdq = 1;
  size_t coff = 0, doff = 0;
  int rc = DN_OK;
  for (int i = 0; i < cfg->n_layers && rc == DN_OK; i++) {
    SeqLayer& l = m->L[i];
    l.c = layers[i];
    memset(l.w, 0, sizeof(l.w));
    memset(l.tm_ok, 0, sizeof(l.tm_ok));
    l.inv_freq = nullptr;
    l.kv_index = -1;
    const dn_seq_layer_cfg& c = l.c;
    if (c.heads <= 0 || c.kv_heads <= 0 || c.heads % c.kv_heads || c.dim <= 0 || c.vdim <= 0) {
      rc = fail(DN_EINVAL, "layer %d: heads %d / kv_heads %d / dim %d / vdim %d unsupported", i, c.heads, c.kv_heads, c.dim, c.vdim);
      break;
    }
    if (c.conv < 0 || c.conv > 9) { rc = fail(DN_EINVAL, "layer %d: conv taps %d unsupported (0..9)", i, c.conv); break; }
    if (c.mixer == DN_MIX_ATTENTION) {
      if (c.vdim > 256) { rc = fail(DN_EINVAL, "layer %d: vdim %d > 256", i, c.vdim); break; }
      if (c.rot_dims < 0 || c.rot_dims > c.dim || (c.rot_dims & 1)) { rc = fail(DN_EINVAL, "layer %d: rot dims %d unsupported", i, c.rot_dims); break; }
      l.Cq = c.heads * c.dim;
      l.Co = c.heads * c.vdim;
      if (c.kv_from >= 0) {
        if (c.kv_from >= i || m->L[c.kv_from].c.mixer != DN_MIX_ATTENTION || m->L[c.kv_from].c.kv_from >= 0 ||
            m->L[c.kv_from].c.kv_heads != c.kv_heads || m->L[c.kv_from].c.dim != c.dim || m->L[c.kv_from].c.vdim != c.vdim) {
          rc = fail(DN_EINVAL, "layer %d: kv_from %d must name an earlier attention layer with its own keys and the same head sizes", i, c.kv_from);
          break;
        }
        l.kv_index = m->L[c.kv_from].kv_index;
        l.Ck = l.Cv = 0;
      } else {
        l.Ck = c.kv_heads * c.dim;
        l.Cv = c.kv_heads * c.vdim;
        l.kv_index = (int)m->kpool.size();
        m->kpool.push_back(nullptr);
        m->vpool.push_back(nullptr);
        if ((rc = dalloc(&m->kpool.back(), (size_t)cfg->pool_pages * PAGE * l.Ck * m->esz)) != DN_OK) break;
        if ((rc = dalloc(&m->vpool.back(), (size_t)cfg->pool_pages * PAGE * l.Cv * m->esz)) != DN_OK) break;
      }
      if (c.rot_dims > 0) {
        std::vector<float> f(c.rot_dims / 2);
        for (int j = 0; j < c.rot_dims / 2; j++) f[j] = (float)std::pow((double)c.rot_base, -2.0 * j / (double)c.rot_dims);
        if ((rc = dalloc(&l.inv_freq, f.size() * 4)) != DN_OK) break;
        if (cudaMemcpy(l.inv_freq, f.data(), f.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess) { rc = fail(DN_ECUDA, "inv_freq upload failed"); break; }
      }
    } else if (c.mixer == DN_MIX_DELTA) {
      if (c.dim > 1024) { rc = fail(DN_EINVAL, "layer %d: delta dim %d > 1024", i, c.dim); break; }
      l.Cq = l.Ck = c.kv_heads * c.dim;
      l.Cv = l.Co = c.heads * c.vdim;
      l.delta_off = doff;
      doff += (size_t)c.heads * c.dim * c.vdim;
      mdq = std::max(mdq, l.Cq);
    } else {
      rc = fail(DN_EINVAL, "layer %d: mixer %d unknown", i, c.mixer);
      break;
    }
    l.conv_off = coff;
    if (c.conv > 1) coff += (size_t)(c.conv - 1) * (l.Cq + l.Ck + l.Cv);
    mq = std::max(mq, l.Cq); mk = std::max(mk, l.Ck); mv = std::max(mv, l.Cv); mo = std::max(mo, l.Co);
    mh = std::max(mh, c.heads); mff = std::max(mff, c.ff);
  }
  const size_t MB = m->MB, W = cfg->width, e = m->esz;
  m->conv_stride = coff;
  m->delta_stride = doff;
#define DA(p, bytes) if (rc == DN_OK) rc = dalloc(&p, (bytes))
  DA(m->xs, (size_t)m->S1 * MB * W * 4); DA(m->y, MB * W * 4); DA(m->pa, MB * mh * 4); DA(m->pb, MB * mh * 4);
  DA(m->qn, MB * mdq * 4); DA(m->kn, MB * mdq * 4); DA(m->vv, MB * mo * 4); DA(m->od, MB * mo * 4);
  DA(m->beta, MB * mh * 4); DA(m->decay, MB * mh * 4);
  DA(m->h, MB * W * e); DA(m->uq, MB * mq * e); DA(m->uk, MB * mk * e); DA(m->uv, MB * mv * e); DA(m->qb, MB * mq * e);
  DA(m->mo, MB * mo * e); DA(m->gt, MB * mo * e); DA(m->act, MB * mff * e);
  DA(m->conv_state, (size_t)cfg->max_seqs * coff * e); DA(m->delta_state, (size_t)cfg->max_seqs * doff * 4);
  m->stage_ints = 4 * MB + 3 * (size_t)(cfg->max_seqs + 1) + MB;
  DA(m->stage_d, m->stage_ints * 4); DA(m->bt_d, (size_t)cfg->max_seqs * m->max_pages * 4); DA(m->tc_err, 16);
  DA(m->lg_buf, (size_t)8 * cfg->vocab * 4);
#undef DA
  if (rc == DN_OK && cudaMemset(m->tc_err, 0, 16) != cudaSuccess) rc = fail(DN_ECUDA, "memset failed");
  if (rc == DN_OK && cfg->dtype == DN_SEQ_BF16) {
    make_xmaps(&m->x_h, m->h, m->MB, cfg->width);
    for (auto& l : m->L) {
      make_xmaps(&l.x_mo, m->mo, m->MB, l.Co);
      if (l.c.ff > 0) make_xmaps(&l.x_act, m->act, m->MB, l.c.ff);
    }
  }
  if (rc == DN_OK && cudaHostAlloc((void**)&m->stage_h, m->stage_ints * 4, cudaHostAllocPortable) != cudaSuccess) rc = fail(DN_ENOMEM, "pinned staging failed");
  if (rc == DN_OK && cudaHostAlloc((void**)&m->bt_h, (size_t)cfg->max_seqs * m->max_pages * 4, cudaHostAllocPortable) != cudaSuccess) rc = fail(DN_ENOMEM, "pinned block table failed");
  if (rc == DN_OK && cudaEventCreateWithFlags(&m->staged, cudaEventDisableTiming) != cudaSuccess) rc = fail(DN_ECUDA, "event creation failed");
  if (rc != DN_OK) { dn_seq_model_destroy(m); return rc; }
  for (int p = cfg->pool_pages - 1; p >= 0; p--) m->free_pages.push_back(p);
  for (int s = cfg->max_seqs - 1; s >= 0; s--) m->free_slots.push_back(s);
  m->pages.resize(cfg->max_seqs);
  m->length.assign(cfg->max_seqs, -1);
  *out = m;
  return DN_OK;
}

extern "C" int dn_seq_bind(dn_seq_model* m, int layer, int which, const void* p) {
  if (!m) return fail(DN_EINVAL, "null model");
  const bool b16 = m->cfg.dtype == DN_SEQ_BF16;
  for (auto& g : m->graphs) cudaGraphExecDestroy(g.second.first);     // captured steps hold the old pointers
  m->graphs.clear();
  if (layer < 0) {
    if (which == DN_SQ_EMBED) m->embed = p;
    else if (which == DN_SQ_FINAL_NORM) m->final_norm = p;
    else if (which == DN_SQ_HEAD) {
      m->head = p;
      m->tm_head_ok = b16 && make_tmap(&m->tm_head, p, m->cfg.vocab, m->cfg.width, dn::TC_BM);
    } else return fail(DN_EINVAL, "tensor %d is not a model tensor", which);
    return DN_OK;
  }
  if (layer >= (int)m->L.size() || which < 0 || which >= DN_SQ_COUNT) return fail(DN_EINVAL, "layer %d / tensor %d out of range", layer, which);
  SeqLayer& l = m->L[layer];
  l.w[which] = p;
  int rows = 0, cols = m->cfg.width;
  switch (which) {
    case DN_SQ_Q: rows = l.Cq; break;
    case DN_SQ_K: rows = l.Ck; break;
    case DN_SQ_V: rows = l.Cv; break;
    case DN_SQ_G: rows = l.Co; break;
    case DN_SQ_A: case DN_SQ_B: rows = l.c.heads; break;
    case DN_SQ_GATE: case DN_SQ_UP: rows = l.c.ff; break;
    case DN_SQ_O: rows = m->cfg.width; cols = l.Co; break;
    case DN_SQ_DOWN: rows = m->cfg.width; cols = l.c.ff; break;
    default: break;
  }
  l.tm_ok[which] = b16 && rows > 0 && make_tmap(&l.tm[which], p, rows, cols, dn::TC_BM);
  return DN_OK;
}

extern "C" int dn_seq_open(dn_seq_model* m, dn_seq_stream s, int* slot_out) {
  if (!m || !slot_out) return fail(DN_EINVAL, "null argument");
  if (m->free_slots.empty()) return fail(DN_ENOSPC, "all %d state slots are in use", m->cfg.max_seqs);
  const int slot = m->free_slots.back();
  // the slot's recurrent state and carried conv inputs start at zero, behind whatever still reads the slot on s
  if (m->conv_stride) CK(cudaMemsetAsync((char*)m->conv_state + (size_t)slot * m->conv_stride * m->esz, 0, m->conv_stride * m->esz, (cudaStream_t)s));
  if (m->delta_stride) CK(cudaMemsetAsync(m->delta_state + (size_t)slot * m->delta_stride, 0, m->delta_stride * 4, (cudaStream_t)s));
  m->free_slots.pop_back();
  m->length[slot] = 0;
  m->pages[slot].clear();
  *slot_out = slot;
  return DN_OK;
}

extern "C" int dn_seq_close(dn_seq_model* m, int slot) {
  if (!m || slot < 0 || slot >= m->cfg.max_seqs || m->length[slot] < 0) return fail(DN_EINVAL, "slot %d is not open", slot);
  for (auto it = m->pages[slot].rbegin(); it != m->pages[slot].rend(); ++it) m->free_pages.push_back(*it);
  m->pages[slot].clear();
  m->length[slot] = -1;
  m->free_slots.push_back(slot);
  return DN_OK;
}

extern "C" int dn_seq_length(dn_seq_model* m, int slot) {
  if (!m || slot < 0 || slot >= m->cfg.max_seqs) return DN_EINVAL;
  return m->length[slot];
}
extern "C" int dn_seq_check(dn_seq_model* m, dn_seq_stream s) {
  if (!m) return fail(DN_EINVAL, "null model");
  unsigned int e = 0;
  CK(cudaMemcpyAsync(&e, m->tc_err, 4, cudaMemcpyDeviceToHost, (cudaStream_t)s));
  CK(cudaStreamSynchronize((cudaStream_t)s));
  if (e) return fail(-62, "a bounded wait inside a GEMM kernel ran out (code %u): results of this model are invalid", e);
  return DN_OK;
}
extern "C" int dn_seq_profile(dn_seq_model* m, int on) {
  if (!m) return fail(DN_EINVAL, "null model");
  m->prof_on = on != 0;
  return DN_OK;
}
extern "C" int dn_seq_profile_read(dn_seq_model* m, double* ms_out, int reset) {
  if (!m || !ms_out) return fail(DN_EINVAL, "bad argument");
  CK(cudaDeviceSynchronize());
  for (size_t i = 0; i + 1 < m->prof_marks.size(); i++) {
    float ms = 0.f;
    // a step's last mark closes it: the gap to the next step's first mark is host time, not a phase
    if (m->prof_marks[i].first != DN_SEQ_PH_OTHER || m->prof_marks[i + 1].first != DN_SEQ_PH_EMBED) {
      CK(cudaEventElapsedTime(&ms, m->prof_marks[i].second, m->prof_marks[i + 1].second));
      m->prof_ms[m->prof_marks[i].first] += ms;
    }
  }
  for (auto& pm : m->prof_marks) m->prof_pool.push_back(pm.second);
  m->prof_marks.clear();
  for (int i = 0; i < DN_SEQ_PH_COUNT; i++) ms_out[i] = m->prof_ms[i];
  if (reset) for (int i = 0; i < DN_SEQ_PH_COUNT; i++) m->prof_ms[i] = 0;
  return DN_OK;
}
extern "C" int dn_seq_free_pages(dn_seq_model* m) { return m ? (int)m->free_pages.size() : DN_EINVAL; }
extern "C" int dn_seq_free_slots(dn_seq_model* m) { return m ? (int)m->free_slots.size() : DN_EINVAL; }

// ---------------------------------------------------------------------------------------------------------------
template <int BN, int EPI, int STAGES>
static cudaError_t launch_tc(const CUtensorMap& w, const CUtensorMap& w2, const CUtensorMap& x, const dn::TcParams& p, cudaStream_t s) {
  constexpr int NA = dn::epi_two_weights(EPI) ? 2 : 1;
  constexpr size_t smem = (size_t)STAGES * (NA * dn::TC_BM * dn::TC_BK * 2 + BN * dn::TC_BK * 2) + 1024 + 256;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(dn::k_gemm_tc<BN, EPI, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr = true;
  }
  const int tiles = ((p.N + dn::TC_BM - 1) / dn::TC_BM) * ((p.T + BN - 1) / BN);
  g_launches++;
  dn::k_gemm_tc<BN, EPI, STAGES><<<tiles < g_sms ? tiles : g_sms, dn::TC_THREADS, smem, s>>>(w, w2, x, p);
  return cudaGetLastError();
}
// token-tile width: the widest that still gives about one CTA per SM
template <int EPI>
static cudaError_t gemm_tc(const CUtensorMap& w, const CUtensorMap& w2, const XMaps& x, const dn::TcParams& p, cudaStream_t s) {
  constexpr bool two = dn::epi_two_weights(EPI);
  const int n_tiles = (p.N + dn::TC_BM - 1) / dn::TC_BM;
  auto tiles = [&](int bn) { return n_tiles * ((p.T + bn - 1) / bn); };
  if (p.T > 64 && tiles(128) >= 100) return launch_tc<128, EPI, (two ? 4 : 6)>(w, w2, x.m[2], p, s);
  if (p.T > 32 && (tiles(64) >= 100 || tiles(64) * 2 > tiles(32))) return launch_tc<64, EPI, (two ? 5 : 8)>(w, w2, x.m[1], p, s);
  return launch_tc<32, EPI, (two ? 5 : 8)>(w, w2, x.m[0], p, s);
}

// One product Y[N, O] = X[N, K] W[O, K]^T (act: gelu_tanh(X W^T) * (X W2^T)).  bf16 batches of 16 tokens and more run on
// the tcgen05 GEMM when the operands have TMA descriptors; a few rows (decode) on the weight-streaming row kernel;
// everything else, and all of fp32, on the CUDA-core tiles.
struct LinMaps { const CUtensorMap* w; const CUtensorMap* w2; const XMaps* x; };
template <class T>
static cudaError_t linear(dn_seq_model* m, cudaStream_t s, const T* X, const void* W, const void* W2, void* Y, int N, int O, int K, bool out32,
                          int act, LinMaps tm = LinMaps{nullptr, nullptr, nullptr}) {
  if (std::is_same<T, bf16>::value && N >= 16 && O >= 32 && tm.w && tm.x && tm.x->ok && (!act || tm.w2)) {
    dn::TcParams p;
    memset(&p, 0, sizeof(p));
    p.T = N; p.N = O; p.K = K; p.ldy = O; p.Y = (dn::bf16*)Y; p.err = m->tc_err;
    if (act) return gemm_tc<dn::EPI_GEGLU>(*tm.w, *tm.w2, *tm.x, p, s);
    if (out32) return gemm_tc<dn::EPI_STORE_F32>(*tm.w, *tm.w, *tm.x, p, s);
    return gemm_tc<dn::EPI_STORE>(*tm.w, *tm.w, *tm.x, p, s);
  }
  if (N <= 8) {
    dim3 grid((O + 7) / 8);
    if (out32) return launch(k_linear_rows<T, true>, grid, dim3(256), 0, s, X, (const T*)W, (const T*)W2, Y, N, O, K, act);
    return launch(k_linear_rows<T, false>, grid, dim3(256), 0, s, X, (const T*)W, (const T*)W2, Y, N, O, K, act);
  }
  dim3 grid((O + 63) / 64, (N + 63) / 64);
  if (out32) return launch(k_linear<T, true>, grid, dim3(256), 0, s, X, (const T*)W, (const T*)W2, Y, N, O, K, act);
  return launch(k_linear<T, false>, grid, dim3(256), 0, s, X, (const T*)W, (const T*)W2, Y, N, O, K, act);
}

// Attention of a step: bf16 steps that bring a prompt portion (an entry of 16 tokens or more) run on the MMA tiles when
// the head sizes fit its templates; decode-only steps, odd head sizes and fp32 on the one-warp-per-(token, head) kernel.
template <class T>
static bool attn_tiles_ok(const dn_seq_layer_cfg& lc, const Batch& b) {
  return std::is_same<T, bf16>::value && b.max_len >= 16 && lc.dim % 8 == 0 && lc.vdim % 8 == 0 && lc.dim <= 128 && lc.vdim <= 128;
}
template <int DKP, int DVP>
static cudaError_t attn_tiles_launch(cudaStream_t s, const Batch& b, const bf16* q, const bf16* kp, const bf16* vp, const dn_seq_layer_cfg& lc,
                                     bf16* out) {
  constexpr size_t smem = ((size_t)2 * AT_ROWS * (DKP + 8) + (size_t)AT_ROWS * (DVP + 8)) * 2;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(k_attn_tiles<DKP, DVP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr = true;
  }
  g_launches++;
  k_attn_tiles<DKP, DVP><<<dim3(b.row_tiles, lc.heads), 128, smem, s>>>(b, q, kp, vp, lc.heads, lc.kv_heads, lc.dim, lc.vdim, lc.chunk, lc.scale, out);
  return cudaGetLastError();
}
static cudaError_t attn_tiles(cudaStream_t s, const Batch& b, const bf16* q, const bf16* kp, const bf16* vp, const dn_seq_layer_cfg& lc, bf16* out) {
  const int kq = lc.dim <= 32 ? 0 : lc.dim <= 64 ? 1 : 2, vq = lc.vdim <= 32 ? 0 : lc.vdim <= 64 ? 1 : 2;
#define AT(a, c, A, Cc) if (kq == a && vq == c) return attn_tiles_launch<A, Cc>(s, b, q, kp, vp, lc, out);
  AT(0, 0, 32, 32) AT(0, 1, 32, 64) AT(0, 2, 32, 128) AT(1, 0, 64, 32) AT(1, 1, 64, 64) AT(1, 2, 64, 128)
  AT(2, 0, 128, 32) AT(2, 1, 128, 64) AT(2, 2, 128, 128)
#undef AT
  return cudaErrorInvalidValue;
}

// phase boundary: the time from this mark to the next one is booked on `phase`
static cudaError_t mark(dn_seq_model* m, int phase, cudaStream_t s) {
  if (!m->prof_on) return cudaSuccess;
  cudaEvent_t ev;
  if (!m->prof_pool.empty()) { ev = m->prof_pool.back(); m->prof_pool.pop_back(); }
  else { cudaError_t e = cudaEventCreate(&ev); if (e != cudaSuccess) return e; }
  m->prof_marks.emplace_back(phase, ev);
  return cudaEventRecord(ev, s);
}

template <class T>
static int step_T(dn_seq_model* m, const Batch& b, int n_want, const int32_t* want_dev, float* logits, float* trace, cudaStream_t s) {
  const dn_seq_cfg& c = m->cfg;
  const int N = b.N, W = c.width, S = c.streams, S1 = m->S1;
  const size_t nsm = ((size_t)W + 40) * 4;
  const int ew = (int)(((size_t)N * W + 255) / 256), ew4 = (int)(((size_t)N * W / 4 + 255) / 256);
  const dim3 nthr(W >= 4096 ? 512 : W >= 2048 ? 256 : 128);     // threads of a norm block: a function of the width only
  auto write_back = [&](const T* mix, const T* out) {
    if (W % 4 == 0) return launch(k_write_back<T, 4>, dim3(ew4), dim3(256), 0, s, m->xs, N, W, S, mix, out, (const float*)m->y);
    return launch(k_write_back<T, 1>, dim3(ew), dim3(256), 0, s, m->xs, N, W, S, mix, out, (const float*)m->y);
  };
#define PH(id) CK(mark(m, id, s))
  PH(DN_SEQ_PH_EMBED);
  CK(launch(k_embed<T>, dim3(N), dim3(128), 0, s, (const T*)m->embed, b, c.embed_scale, W, S1, m->xs));
  for (int li = 0; li < c.n_layers; li++) {
    SeqLayer& l = m->L[li];
    const dn_seq_layer_cfg& lc = l.c;
    auto w = [&](int i) { return (const T*)l.w[i]; };
    // ---- mixer sublayer
    PH(DN_SEQ_PH_NORM);
    CK(launch(k_read_norm<T>, dim3(N), nthr, nsm, s, m->xs, N, W, S, w(DN_SQ_HC1_IN), w(DN_SQ_NORM1), 1, 0, c.eps, (const int32_t*)nullptr, (T*)m->h));
    T* cst = (T*)m->conv_state + l.conv_off;
    auto wm = [&](int i) { return l.tm_ok[i] ? &l.tm[i] : (const CUtensorMap*)nullptr; };
    PH(DN_SEQ_PH_PROJ);
    const bool few = N <= 8;      // a decode step: all projections of the mixer in one launch of the row kernel
    if (few) {
      LinSegs sg;
      memset(&sg, 0, sizeof(sg));
      auto add = [&](int which, void* y, int rows, int o32) {
        if (rows <= 0) return;
        sg.W[sg.n] = l.w[which]; sg.Y[sg.n] = y; sg.O[sg.n] = rows; sg.out32[sg.n] = o32; sg.n++;
      };
      add(DN_SQ_Q, m->uq, l.Cq, 0); add(DN_SQ_K, m->uk, l.Ck, 0); add(DN_SQ_V, m->uv, l.Cv, 0);
      if (lc.mixer == DN_MIX_DELTA) { add(DN_SQ_A, m->pa, lc.heads, 1); add(DN_SQ_B, m->pb, lc.heads, 1); add(DN_SQ_G, m->gt, l.Co, 0); }
      int blocks = 0;
      for (int i = 0; i < sg.n; i++) blocks += (sg.O[i] + 7) / 8;
      CK(launch(k_linear_rows_multi<T>, dim3(blocks), dim3(256), 0, s, (const T*)m->h, sg, N, W));
    } else {
      CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_Q], nullptr, m->uq, N, l.Cq, W, false, 0, LinMaps{wm(DN_SQ_Q), nullptr, &m->x_h}));
      if (l.Ck) CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_K], nullptr, m->uk, N, l.Ck, W, false, 0, LinMaps{wm(DN_SQ_K), nullptr, &m->x_h}));
      if (l.Cv) CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_V], nullptr, m->uv, N, l.Cv, W, false, 0, LinMaps{wm(DN_SQ_V), nullptr, &m->x_h}));
    }
    if (lc.mixer == DN_MIX_ATTENTION) {
      AttnPrep a{lc.heads, lc.kv_heads, lc.dim, lc.vdim, lc.conv, lc.rot_dims, l.Ck ? 1 : 0, c.eps, l.inv_freq};
      const size_t sm = ((size_t)l.Cq + l.Ck + 40) * 4;
      PH(DN_SEQ_PH_ATTN_PREP);
      CK(launch(k_attn_prep<T>, dim3(N), dim3(256), sm, s, a, b, (const T*)m->uq, (const T*)m->uk, (const T*)m->uv, w(DN_SQ_Q_CONV),
                w(DN_SQ_K_CONV), w(DN_SQ_V_CONV), w(DN_SQ_Q_NORM), w(DN_SQ_K_NORM), (const T*)cst, m->conv_stride, (T*)m->qb,
                (T*)m->kpool[l.kv_index], (T*)m->vpool[l.kv_index]));
      PH(DN_SEQ_PH_ATTN);
      if (attn_tiles_ok<T>(lc, b))
        CK(attn_tiles(s, b, (const bf16*)m->qb, (const bf16*)m->kpool[l.kv_index], (const bf16*)m->vpool[l.kv_index], lc, (bf16*)m->mo));
      else
        CK(launch(k_attn<T>, dim3(N, lc.heads), dim3(AT_WARPS * 32), (size_t)(((lc.dim + 3) & ~3) + AT_WARPS * (2 + (lc.vdim + 31) / 32 * 32)) * 4, s, b,
                  (const T*)m->qb, (const T*)m->kpool[l.kv_index],
                  (const T*)m->vpool[l.kv_index], lc.heads, lc.kv_heads, lc.dim, lc.vdim, lc.chunk, lc.scale, (T*)m->mo));
    } else {
      if (!few) {
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_A], nullptr, m->pa, N, lc.heads, W, true, 0, LinMaps{wm(DN_SQ_A), nullptr, &m->x_h}));
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_B], nullptr, m->pb, N, lc.heads, W, true, 0, LinMaps{wm(DN_SQ_B), nullptr, &m->x_h}));
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_G], nullptr, m->gt, N, l.Co, W, false, 0, LinMaps{wm(DN_SQ_G), nullptr, &m->x_h}));
      }
      DeltaPrep a{lc.heads, lc.kv_heads, lc.dim, lc.vdim, lc.conv};
      PH(DN_SEQ_PH_DELTA_PREP);
      CK(launch(k_delta_prep<T>, dim3(N), dim3(256), (size_t)2 * l.Cq * 4, s, a, b, (const T*)m->uq, (const T*)m->uk, (const T*)m->uv,
                w(DN_SQ_Q_CONV), w(DN_SQ_K_CONV), w(DN_SQ_V_CONV), (const float*)m->pa, (const float*)m->pb, w(DN_SQ_A_LOG),
                w(DN_SQ_DT_BIAS), (const T*)cst, m->conv_stride, m->qn, m->kn, m->vv, m->beta, m->decay));
      // rows a lane (R) and lanes a column (P): the smallest P R >= dk of this table
      static const int RP[8][3] = {{8, 8, 1}, {16, 8, 2}, {32, 8, 4}, {64, 8, 8}, {128, 16, 8}, {256, 16, 16}, {512, 16, 32}, {1024, 32, 32}};
      int R = 32, P = 32;
      for (int i = 7; i >= 0; i--) if (lc.dim <= RP[i][0]) { R = RP[i][1]; P = RP[i][2]; }
      dim3 grid(b.E * lc.heads, (lc.vdim + 31) / 32);
      float* st = m->delta_state + l.delta_off;
      // tokens per staged tile: two tiles of `per` floats a token within ~36 KB of shared memory
      const int per = 2 * P * (R + 4) + 36, TB = std::max(1, std::min(16, 4500 / per));
      const size_t dsm = (size_t)2 * TB * per * 4;
#define DR(Rv, Pv) if (R == Rv && P == Pv) CK(launch(k_delta_rule<Rv, Pv>, grid, dim3(32 * Pv), dsm, s, b, lc.heads, lc.kv_heads, lc.dim, lc.vdim, TB, \
                         (const float*)m->qn, (const float*)m->kn, (const float*)m->vv, (const float*)m->beta, (const float*)m->decay, st,      \
                         m->delta_stride, m->od))
      PH(DN_SEQ_PH_DELTA_RULE);
      DR(8, 1); DR(8, 2); DR(8, 4); DR(8, 8); DR(16, 8); DR(16, 16); DR(16, 32); DR(32, 32);
#undef DR
      PH(DN_SEQ_PH_DELTA_OUT);
      CK(launch(k_delta_out<T>, dim3(N, lc.heads), dim3(32), 0, s, (const float*)m->od, (const T*)m->gt, w(DN_SQ_OUT_NORM), lc.heads, lc.vdim,
                c.eps, (T*)m->mo));
    }
    if (lc.conv > 1) {
      PH(DN_SEQ_PH_CARRY);
      CarrySrc<T> cs{{(const T*)m->uq, (const T*)m->uk, (const T*)m->uv}, {l.Cq, l.Ck, l.Cv}};
      CK(launch(k_conv_carry<T>, dim3((std::max(l.Cq, std::max(l.Ck, l.Cv)) + 127) / 128, b.E, 3), dim3(128), 0, s, cs, lc.conv, b, cst, m->conv_stride));
    }
    PH(DN_SEQ_PH_OUT_PROJ);
    CK(linear<T>(m, s, (const T*)m->mo, l.w[DN_SQ_O], nullptr, m->y, N, W, l.Co, true, 0, LinMaps{wm(DN_SQ_O), nullptr, &l.x_mo}));
    PH(DN_SEQ_PH_WRITE_BACK);
    CK(write_back(w(DN_SQ_HC1_MIX), w(DN_SQ_HC1_OUT)));
    // ---- feed-forward sublayer
    if (lc.ff > 0) {
      PH(DN_SEQ_PH_NORM);
      CK(launch(k_read_norm<T>, dim3(N), nthr, nsm, s, m->xs, N, W, S, w(DN_SQ_HC2_IN), w(DN_SQ_NORM2), 1, 0, c.eps, (const int32_t*)nullptr, (T*)m->h));
      PH(DN_SEQ_PH_FF_UP);
      CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_GATE], l.w[DN_SQ_UP], m->act, N, lc.ff, W, false, 1, LinMaps{wm(DN_SQ_GATE), wm(DN_SQ_UP), &m->x_h}));
      PH(DN_SEQ_PH_FF_DOWN);
      CK(linear<T>(m, s, (const T*)m->act, l.w[DN_SQ_DOWN], nullptr, m->y, N, W, lc.ff, true, 0, LinMaps{wm(DN_SQ_DOWN), nullptr, &l.x_act}));
      PH(DN_SEQ_PH_WRITE_BACK);
      CK(write_back(w(DN_SQ_HC2_MIX), w(DN_SQ_HC2_OUT)));
    }
    PH(DN_SEQ_PH_OTHER);
    if (trace) CK(launch(k_stream_sum, dim3(ew), dim3(256), 0, s, (const float*)m->xs, N, W, S1, trace + (size_t)li * N * W));
  }
  if (n_want > 0) {
    PH(DN_SEQ_PH_NORM);
    CK(launch(k_read_norm<T>, dim3(n_want), nthr, nsm, s, m->xs, N, W, S, (const T*)nullptr, (const T*)m->final_norm, 1, 1, c.eps, want_dev, (T*)m->h));
    PH(DN_SEQ_PH_HEAD);
    CK(linear<T>(m, s, (const T*)m->h, m->head, nullptr, logits, n_want, c.vocab, W, true, 0, LinMaps{m->tm_head_ok ? &m->tm_head : nullptr, nullptr, &m->x_h}));
  }
  PH(DN_SEQ_PH_OTHER);
#undef PH
  return DN_OK;
}

extern "C" int dn_seq_step(dn_seq_model* m, int E, const int32_t* slots, const int32_t* counts, const int32_t* tokens, int n_want,
                           const int32_t* want, float* logits, float* trace, dn_seq_stream sp) {
  if (!m || E <= 0 || !slots || !counts || !tokens || (n_want > 0 && (!want || !logits))) return fail(DN_EINVAL, "bad argument");
  if (E > m->cfg.max_seqs) return fail(DN_EINVAL, "%d entries > %d state slots", E, m->cfg.max_seqs);
  cudaStream_t s = (cudaStream_t)sp;
  int N = 0;
  size_t need = 0;
  for (int e = 0; e < E; e++) {
    const int sl = slots[e];
    if (sl < 0 || sl >= m->cfg.max_seqs || m->length[sl] < 0) return fail(DN_EINVAL, "entry %d: slot %d is not open", e, sl);
    for (int f = 0; f < e; f++) if (slots[f] == sl) return fail(DN_EINVAL, "slot %d appears twice in one step", sl);
    if (counts[e] <= 0) return fail(DN_EINVAL, "entry %d brings no tokens", e);
    N += counts[e];
    const size_t pages = ((size_t)m->length[sl] + counts[e] + PAGE - 1) / PAGE;
    if (pages > (size_t)m->max_pages) return fail(DN_ENOSPC, "sequence too long for the block table");
    if (pages > m->pages[sl].size()) need += pages - m->pages[sl].size();
  }
  if (N > m->MB) return fail(DN_EINVAL, "%d tokens > max_batch_tokens %d", N, m->MB);
  if (n_want > N) return fail(DN_EINVAL, "more wanted rows than tokens");
  for (int i = 0; i < N; i++) if (tokens[i] < 0 || tokens[i] >= m->cfg.vocab) return fail(DN_EINVAL, "token id %d out of range", tokens[i]);
  if (need > m->free_pages.size()) return fail(DN_ENOSPC, "cache pool exhausted: %zu pages needed, %zu free", need, m->free_pages.size());
  for (int i = 0; i < n_want; i++) if (want[i] < 0 || want[i] >= N) return fail(DN_EINVAL, "wanted row %d out of range", want[i]);
  if (!m->embed || !m->final_norm || !m->head) return fail(DN_ENOENT, "embedding / final norm / head are not bound");
  for (int i = 0; i < m->cfg.n_layers; i++) {
    const SeqLayer& l = m->L[i];
    auto has = [&](int k) { return l.w[k] != nullptr; };
    bool ok = has(DN_SQ_NORM1) && has(DN_SQ_Q) && has(DN_SQ_O) && (l.c.ff == 0 || (has(DN_SQ_NORM2) && has(DN_SQ_GATE) && has(DN_SQ_UP) && has(DN_SQ_DOWN)));
    if (l.Ck) ok = ok && has(DN_SQ_K) && has(DN_SQ_V);
    if (l.c.conv > 0) ok = ok && has(DN_SQ_Q_CONV) && (!l.Ck || (has(DN_SQ_K_CONV) && has(DN_SQ_V_CONV)));
    if (l.c.mixer == DN_MIX_ATTENTION) ok = ok && has(DN_SQ_Q_NORM) && (!l.Ck || has(DN_SQ_K_NORM));
    else ok = ok && has(DN_SQ_A) && has(DN_SQ_B) && has(DN_SQ_G) && has(DN_SQ_A_LOG) && has(DN_SQ_DT_BIAS) && has(DN_SQ_OUT_NORM);
    if (m->cfg.streams > 0) ok = ok && has(DN_SQ_HC1_IN) && has(DN_SQ_HC1_OUT) && has(DN_SQ_HC1_MIX) &&
                                 (l.c.ff == 0 || (has(DN_SQ_HC2_IN) && has(DN_SQ_HC2_OUT) && has(DN_SQ_HC2_MIX)));
    if (!ok) return fail(DN_ENOENT, "layer %d: not every tensor of the layer is bound", i);
  }
  // the previous step's staging copies must have read the pinned buffers before they are rewritten
  CK(cudaEventSynchronize(m->staged));
  int32_t* h = m->stage_h;
  int32_t *tok = h, *slot = h + N, *pos = h + 2 * N, *first = h + 3 * N, *es = h + 4 * N, *esl = es + E + 1, *ep0 = esl + E, *wr = ep0 + E;
  int n = 0;
  for (int e = 0; e < E; e++) {
    const int sl = slots[e];
    const size_t pages = ((size_t)m->length[sl] + counts[e] + PAGE - 1) / PAGE;
    const size_t had = m->pages[sl].size();
    while (m->pages[sl].size() < pages) {
      const int pg = m->free_pages.back();
      m->free_pages.pop_back();
      m->bt_h[(size_t)sl * m->max_pages + m->pages[sl].size()] = pg;
      m->pages[sl].push_back(pg);
    }
    if (pages > had)
      CK(cudaMemcpyAsync(m->bt_d + (size_t)sl * m->max_pages + had, m->bt_h + (size_t)sl * m->max_pages + had, (pages - had) * 4,
                         cudaMemcpyHostToDevice, s));
    es[e] = n; esl[e] = sl; ep0[e] = m->length[sl];
    for (int i = 0; i < counts[e]; i++, n++) { tok[n] = tokens[n]; slot[n] = sl; pos[n] = m->length[sl] + i; first[n] = es[e]; }
    m->length[sl] += counts[e];
  }
  es[E] = N;
  for (int i = 0; i < n_want; i++) wr[i] = want[i];
  const size_t ints = 4 * (size_t)N + 3 * (size_t)E + 1 + n_want;
  CK(cudaMemcpyAsync(m->stage_d, h, ints * 4, cudaMemcpyHostToDevice, s));
  CK(cudaEventRecord(m->staged, s));
  int32_t* d = m->stage_d;
  int max_len = 0, row_tiles = 0;
  for (int e = 0; e < E; e++) { max_len = counts[e] > max_len ? counts[e] : max_len; row_tiles += (counts[e] + AT_ROWS - 1) / AT_ROWS; }
  Batch b{d, d + N, d + 2 * N, d + 3 * N, d + 4 * N, d + 4 * N + E + 1, d + 4 * N + 2 * E + 1, m->bt_d, N, E, m->max_pages, max_len, row_tiles};
  const int32_t* want_dev = d + 4 * N + 3 * E + 1;
  auto run = [&](float* lg) {
    if (m->cfg.dtype == DN_SEQ_F32) return step_T<float>(m, b, n_want, want_dev, lg, trace, s);
    return step_T<bf16>(m, b, n_want, want_dev, lg, trace, s);
  };
  // (the legacy default stream cannot be captured: steps queued on it are launched one by one)
  const bool capturable = s != nullptr && s != cudaStreamLegacy && s != cudaStreamPerThread;
  if (!(m->graphs_on && capturable && N == E && N <= 8 && !trace && !m->prof_on)) return run(logits);
  // a decode step: replay (capturing at first use) the step's kernels as one graph
  const auto key = std::make_pair(E, n_want);
  auto it = m->graphs.find(key);
  if (it == m->graphs.end()) {
    const long long l0 = g_launches.load();
    if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
      cudaGetLastError();          // this stream cannot be captured now (e.g. it is part of the caller's own capture): launch one by one
      return run(logits);
    }
    const int rc = run(m->lg_buf);
    cudaGraph_t graph = nullptr;
    const cudaError_t ec = cudaStreamEndCapture(s, &graph);
    if (rc != DN_OK) { if (graph) cudaGraphDestroy(graph); return rc; }
    if (ec != cudaSuccess) return fail(DN_ECUDA, "graph capture of a decode step failed: %s", cudaGetErrorString(ec));
    cudaGraphExec_t exec = nullptr;
    const cudaError_t ei = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ei != cudaSuccess) return fail(DN_ECUDA, "graph instantiation failed: %s", cudaGetErrorString(ei));
    const long long per = g_launches.load() - l0;
    g_launches -= per;          // captured, not run: replays are what is counted
    it = m->graphs.emplace(key, std::make_pair(exec, per)).first;
  }
  CK(cudaGraphLaunch(it->second.first, s));
  g_launches += it->second.second;
  if (n_want > 0) CK(cudaMemcpyAsync(logits, m->lg_buf, (size_t)n_want * m->cfg.vocab * 4, cudaMemcpyDeviceToDevice, s));
  return DN_OK;
}

extern "C" int dn_seq_set_graphs(dn_seq_model* m, int on) {
  if (!m) return fail(DN_EINVAL, "null model");
  m->graphs_on = on != 0;
  return DN_OK;
}
