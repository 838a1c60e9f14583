// Test infrastructure: the reference-side binding of libfl_b200.so, compiled against the
// reference's own headers. It is the translation unit a maintainer adds in place of
// src/runtime/gpu_exec.cu: the six backend functions declared in
// src/runtime/runtime_internal.h:288-301 keep their C++ names and signatures (so
// src/runtime/runtime.cpp:123-311 links unchanged) and forward to the C ABI of
// include/fl_b200.h. oracle/Makefile compiles it with -DFASTLLM_CUDA and links it against
// the library, which proves the signatures and the symbol set; nothing here runs in a test.
//
// Two more hooks, gpu_plan / gpu_run, hand a frozen task table over as a whole: the place to call
// them is Runtime::run (src/runtime/runtime.cpp:178-292) in a build that replays the table as one
// CUDA graph instead of feeding the reference's task queue.
#include "fl_b200.h"
#include "runtime_internal.h"

#include <cstdio>
#include <cstdlib>

namespace fastllm {
namespace {

fl_b200_ctx *g_ctx = nullptr;
fl_b200_plan *g_plan = nullptr;

[[noreturn]] void die_b200(const char *what) {   // the reference's convention: print and abort (gpu_exec.cu:15-17)
    std::fprintf(stderr, "fastllm/b200: %s: %s\n", what, fl_b200_last_error());
    std::abort();
}
#define B200(call)                               \
    do {                                         \
        if ((call) != FL_B200_OK) die_b200(#call); \
    } while (0)

} // namespace

void *gpu_make_stream() {
    if (!g_ctx) B200(fl_b200_create(/*device=*/0, &g_ctx));
    return fl_b200_stream(g_ctx);
}

int gpu_default_blocks() { return g_ctx ? fl_b200_sm_count(g_ctx) : 148; }
int gpu_resident_blocks(int /*threads*/) { return gpu_default_blocks(); }

// Nothing persistent to start: launches are made per run. The block count is still published where the
// reference's metrics read it (RtShared::gpu_blocks).
int gpu_start(RtShared *sh, int blocks, int /*threads*/, void * /*stream*/, size_t /*persist_bytes*/) {
    const int n = blocks < gpu_default_blocks() ? blocks : gpu_default_blocks();
    if (sh) sh->gpu_blocks = (uint32_t)n;
    return n;
}

void gpu_stop_sync(void * /*stream*/) {
    if (!g_ctx) return;
    B200(fl_b200_sync(g_ctx));
    if (g_plan) { fl_b200_plan_destroy(g_plan); g_plan = nullptr; }
    fl_b200_destroy(g_ctx);
    g_ctx = nullptr;
}

int64_t gpu_calibrate_clock(RtShared * /*sh*/, void * /*stream*/) { return 0; }   // no device-side timestamps are exported

// ---- whole-table hand-over (new hooks) ----
void gpu_plan(const Task *tasks, uint32_t n) {   // once, after Graph::freeze
    static_assert(sizeof(Task) == sizeof(fl_b200_task), "Task layout");
    if (g_plan) { fl_b200_plan_destroy(g_plan); g_plan = nullptr; }
    B200(fl_b200_plan_create(g_ctx, reinterpret_cast<const fl_b200_task *>(tasks), n, &g_plan));
}
void gpu_run() {                                 // inside Runtime::run
    B200(fl_b200_plan_run(g_plan));
    B200(fl_b200_sync(g_ctx));
}
void gpu_exec_task(const Task &t) {              // one task at a time (exec_task_block's role, gpu_exec.cu:64-66)
    B200(fl_b200_exec_task(g_ctx, reinterpret_cast<const fl_b200_task *>(&t)));
    uint32_t st = 0;
    B200(fl_b200_device_status(g_ctx, &st));
    if (st != 0) die_b200("device status");
}

} // namespace fastllm
