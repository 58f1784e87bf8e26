// C ABI of libzb_host.so: CPU-side runtime pieces written in C++ (file streaming for
// the weight loader, span tracer, BPE tokenizer core, /proc + NVML sampling).
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- file streaming ---------------------------------------------------------
// Reads `n` byte ranges (offsets[i], lengths[i]) of the file behind `fd` into `dst`
// back to back, using up to `threads` reader threads.  Returns bytes read or -errno.
long long zbh_pread_spans(int fd, const long long* offsets, const long long* lengths, int n,
                          void* dst, int threads);

// ---- tracer -----------------------------------------------------------------
// Host trace spans recorded into a per-process ring buffer and written as Chrome /
// Perfetto trace-event JSON; optionally mirrored as NVTX ranges when libnvToolsExt
// or the NVTX3 injection is present.
int zbh_trace_start(size_t capacity_events);
int zbh_trace_stop(void);
unsigned long long zbh_trace_begin(const char* name);          // returns a span id
void zbh_trace_end(unsigned long long span_id);
void zbh_trace_instant(const char* name);
long long zbh_trace_count(void);
int zbh_trace_write_json(const char* path);

#ifdef __cplusplus
}
#endif
