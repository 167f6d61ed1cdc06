/* Measurement hooks of libnsa_b200: NOT part of the operator interface (include/nsa_b200.h), which is stateless.  These
 * keep process-wide counters and CUDA events and exist for the benchmark and the tests; a caller of the operators never
 * needs them.  No counterpart in the reference. */
#ifndef NSA_B200_INSTRUMENT_H_
#define NSA_B200_INSTRUMENT_H_

#ifdef __cplusplus
extern "C" {
#endif

/* Number of kernels this library has launched in the calling process.  No counterpart in the reference. */
long long nsa_launch_count(void);

/* Per-kernel device timing: while enabled, every kernel launch is bracketed by CUDA events on its stream.
 * nsa_profile_collect synchronises the device and writes one line "kernel launches total_ms" per kernel for
 * the launches recorded since the previous collect (returns the bytes written).  No counterpart in the reference. */
int nsa_profile_enable(int on);
int nsa_profile_collect(char* buf, int buflen);

#ifdef __cplusplus
}
#endif
#endif /* NSA_B200_INSTRUMENT_H_ */
