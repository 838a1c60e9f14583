// Test infrastructure. Compile-time proof that the task record and parameter
// blocks declared in include/fl_b200.h are field-for-field images of the
// reference's (include/fastllm/fastllm.h:65-97, src/runtime/decode_params.h:23-97).
// Built into oracle/_ref/libflref.so by oracle/Makefile; a layout drift in
// either header stops that build.
#include "fastllm/fastllm.h"
#include "decode_params.h"
#include "../include/fl_b200.h"
#include <cstddef>

using fastllm::Task;

#define SAME_FIELD(f) static_assert(offsetof(Task, f) == offsetof(fl_b200_task, f), "Task::" #f " offset")
static_assert(sizeof(Task) == sizeof(fl_b200_task), "Task size");
static_assert(alignof(Task) == alignof(fl_b200_task), "Task alignment");
SAME_FIELD(id); SAME_FIELD(kind); SAME_FIELD(affinity); SAME_FIELD(fmt); SAME_FIELD(n_consumers);
SAME_FIELD(consumers); SAME_FIELD(w); SAME_FIELD(w_bytes); SAME_FIELD(x); SAME_FIELD(y); SAME_FIELD(rows);
SAME_FIELD(cols); SAME_FIELD(dep_init); SAME_FIELD(dep_count); SAME_FIELD(epoch); SAME_FIELD(handoff_ts);
SAME_FIELD(aux); SAME_FIELD(aux2); SAME_FIELD(nx); SAME_FIELD(xstride); SAME_FIELD(ystride);

static_assert((int)fastllm::TaskKind::STREAM_DOT == FL_B200_STREAM_DOT, "kind");
static_assert((int)fastllm::TaskKind::SIGNAL == FL_B200_SIGNAL, "kind");
static_assert((int)fastllm::TaskKind::RMSNORM == FL_B200_RMSNORM, "kind");
static_assert((int)fastllm::TaskKind::ADD2 == FL_B200_ADD2, "kind");
static_assert((int)fastllm::TaskKind::SILU_MUL == FL_B200_SILU_MUL, "kind");
static_assert((int)fastllm::TaskKind::WMERGE == FL_B200_WMERGE, "kind");
static_assert(fastllm::kNumTaskKinds == FL_B200_ATTN_GQA_F16, "appended kinds start after the reference's");
static_assert((int)fastllm::Fmt::Q4_K == FL_B200_Q4_K && (int)fastllm::Fmt::Q6_K == FL_B200_Q6_K &&
              (int)fastllm::Fmt::Q8_0 == FL_B200_Q8_0 && (int)fastllm::Fmt::Q5_0 == FL_B200_Q5_0 &&
              (int)fastllm::Fmt::F32 == FL_B200_F32, "format ids");

static_assert(sizeof(fastllm::RmsNormP) == sizeof(fl_b200_rmsnorm_p), "RmsNormP");
static_assert(offsetof(fastllm::RmsNormP, eps) == offsetof(fl_b200_rmsnorm_p, eps), "RmsNormP::eps");
static_assert(offsetof(fastllm::RmsNormP, n) == offsetof(fl_b200_rmsnorm_p, n), "RmsNormP::n");
static_assert(sizeof(fastllm::Add2P) == sizeof(fl_b200_add2_p), "Add2P");
static_assert(offsetof(fastllm::Add2P, n) == offsetof(fl_b200_add2_p, n), "Add2P::n");
static_assert(sizeof(fastllm::RouterP) == sizeof(fl_b200_router_p), "RouterP");
static_assert(offsetof(fastllm::RouterP, ids) == offsetof(fl_b200_router_p, ids), "RouterP::ids");
static_assert(offsetof(fastllm::RouterP, top_k) == offsetof(fl_b200_router_p, top_k), "RouterP::top_k");
static_assert(offsetof(fastllm::RouterP, scale) == offsetof(fl_b200_router_p, scale), "RouterP::scale");
static_assert(sizeof(fastllm::WmergeP) == sizeof(fl_b200_wmerge_p), "WmergeP");
static_assert(offsetof(fastllm::WmergeP, y) == offsetof(fl_b200_wmerge_p, y), "WmergeP::y");
static_assert(offsetof(fastllm::WmergeP, scale) == offsetof(fl_b200_wmerge_p, scale), "WmergeP::scale");
static_assert(offsetof(fastllm::WmergeP, n_full) == offsetof(fl_b200_wmerge_p, n_full), "WmergeP::n_full");
static_assert((int)fastllm::TaskKind::STREAM_DOT_IDX == FL_B200_STREAM_DOT_IDX, "kind");
static_assert((int)fastllm::TaskKind::ROUTER_SEL == FL_B200_ROUTER_SEL, "kind");
static_assert(sizeof(fastllm::SiluMulP) == sizeof(fl_b200_silu_mul_p), "SiluMulP");
static_assert(offsetof(fastllm::SiluMulP, n) == offsetof(fl_b200_silu_mul_p, n), "SiluMulP::n");

extern "C" int flref_abi_checked(void) { return 1; }
