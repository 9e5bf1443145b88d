/* TEST INFRASTRUCTURE — exports the reference's own static C functions ref_q4k_dot / ref_q6k_dot
 * (extracted at build time from the reference checkout into _ref/ref_kq_extract.inc by the
 * Makefile) so the oracle can be checked against them. */
#include <stdint.h>
#include <string.h>
#include "ref_kq_extract.inc"

float refkq_q4k_dot(const uint8_t *row, const int8_t *xq, const float *xs, const int32_t *xsum, int cols) { return ref_q4k_dot(row, xq, xs, xsum, cols); }
float refkq_q6k_dot(const uint8_t *row, const int8_t *xq, const float *xs, int cols) { return ref_q6k_dot(row, xq, xs, cols); }
float refkq_half2f(uint16_t h) { return half2f(h); }
