// Cycle-counter and event-trace hooks of the forward attention kernel. They expand to nothing
// unless the file is compiled with -DB200NA_PROFILE=1|2 (never in the product build): level 1
// keeps per-role cycle counters of one softmax thread per half, level 2 adds an event trace of
// the MMA-issuing and load threads in shared memory. The instrumented build also exports
// b200na_debug_set_prof() to hand the kernel a device buffer for the counters.
#pragma once

#ifdef B200NA_PROFILE
#define TRACE(role, code) { if (blockIdx.x == 0 && trace_n_ < 1024) { p.prof[296 * 32 + (role) * 1024 + trace_n_] = (clock64() << 8) | (code); ++trace_n_; } }
#define PROF_DECL int trace_n_ = 0; long long prof_[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long prof_t_ = clock64(); const long long prof_t0_ = prof_t_;
#define PROF_MARK(i) { const long long n_ = clock64(); prof_[i] += n_ - prof_t_; prof_t_ = n_; }
#define PROF_FLUSH(role) { prof_[7] = clock64() - prof_t0_; for (int i_ = 0; i_ < 8; ++i_) p.prof[((long long)blockIdx.x * 4 + (role)) * 8 + i_] = prof_[i_]; }
#if B200NA_PROFILE >= 2
// MMA / load threads: one 32-bit clock read and one shared-memory store per event (anything
// heavier perturbs the single issuing thread); block 0 copies the ring to global at teardown.
#define TRACE2(role, code) { if (trace2_n_ < 1024) { trace2_buf_[((role) - 2) * 1024 + trace2_n_] = ((uint32_t)clock() << 5) | (code); ++trace2_n_; } }
#define PROF2_DECL int trace2_n_ = 0; uint32_t* trace2_buf_ = reinterpret_cast<uint32_t*>(smem + SM::kBytes);
#define PROF2_MARK(i) {}
#define PROF2_FLUSH(role) {}
#else
#define TRACE2(role, code) {}
#define PROF2_DECL
#define PROF2_MARK(i) {}
#define PROF2_FLUSH(role) {}
#endif
#else
#define TRACE2(role, code) {}
#define PROF2_DECL
#define PROF2_MARK(i) {}
#define PROF2_FLUSH(role) {}
#define TRACE(role, code) {}
#define PROF_DECL
#define PROF_MARK(i) {}
#define PROF_FLUSH(role) {}
#endif

