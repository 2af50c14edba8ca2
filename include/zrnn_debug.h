/*
 * zrnn_debug.h - developer aids of libzrnn.so (no counterpart in the reference; not part of the drop-in
 * interface of zrnn.h).  Device-side timelines of the tensor-core kernels, written as %globaltimer values (ns).
 */
#ifndef ZRNN_DEBUG_H
#define ZRNN_DEBUG_H

#ifdef __cplusplus
extern "C" {
#endif

/* Device-side phase stamps of the split-K tensor-core launches.
 * zrnn_debug_tc_profile(d_buf): while d_buf is set, every CTA of every split-K tensor-core launch writes 8
 * %globaltimer values (ns) to d_buf[cta * 8 ..]: start, set-up done, accumulators complete, partial tile pushed,
 * cluster barrier passed, exchange slots read, gate math done, stores issued.  d_buf must hold 8 values per CTA of
 * the largest launch; NULL switches it off.
 * zrnn_debug_tc_timeline(d_buf, slots): launch i (counted from the call) writes the same 8 stamps of its CTA (0,0,0)
 * to d_buf[i * 8 ..] for i < slots. */
int zrnn_debug_tc_profile(long long* d_buf);
int zrnn_debug_tc_timeline(long long* d_buf, int slots);

/* zrnn_debug_decoder_timeline(d_buf, cta): CTA `cta` of every launch of the persistent decoder kernel writes 8 stamps
 * per phase to d_buf[phase * 8 ..]: phase entered, accumulators complete, cluster ready, partial tile pushed,
 * exchange complete, results stored, earlier phases seen complete, phase counted.  d_buf holds 8 values for each of
 * T * (L + 2 or 3) phases; NULL switches it off.  cta < 0: every CTA writes, CTA c to d_buf[(c * phases + phase) * 8 ..]. */
int zrnn_debug_decoder_timeline(long long* d_buf, int cta);

/* Exercise of the bounded device waits: launches one warp that waits on a barrier nothing will ever complete, with a
 * limit of limit_cycles SM cycles (2e6 is about a millisecond).  The wait gives up, the kernel returns, and the device
 * error word holds role 77: zrnn_tc_error() returns it, and the next model-level call that ends with a host
 * synchronisation returns ZRNN_E_TIMEOUT once; the context stays usable. */
int zrnn_debug_bounded_wait(long long limit_cycles, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ZRNN_DEBUG_H */
