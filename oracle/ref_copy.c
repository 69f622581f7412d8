/* Thin exports of the reference's OWN host-side LMAD copy (rts/c/copy.h), compiled from the
 * header where it lies in the reference checkout (never copied into this repository).
 * TEST INFRASTRUCTURE ONLY: the parity tests of the strided-copy entry point compare against
 * it, and check that this repository's classification of a copy (batched transposition / flat
 * copy / general copy) agrees with the reference's.
 *
 * Built by oracle/build.py into oracle/_ref/libref_copy.so when the reference checkout is
 * present; its rts/c directory is given with -I, so the include below resolves to the
 * reference's file.  The header expects a context with a logging switch; the stand-in below
 * keeps logging off.
 */
#include <stdbool.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

struct futhark_context { int logging; FILE *log; };

#include "copy.h"

static struct futhark_context quiet = {0, NULL};

#define EXPORT_COPY(NAME, T)                                                                        \
  void ref_lmad_copy_##NAME(int r, T *dst, int64_t dst_offset, int64_t *dst_strides, T *src,        \
                            int64_t src_offset, int64_t *src_strides, int64_t *shape) {             \
    lmad_copy_##NAME(&quiet, r, dst, dst_offset, dst_strides, src, src_offset, src_strides, shape); \
  }
EXPORT_COPY(1b, uint8_t)
EXPORT_COPY(2b, uint16_t)
EXPORT_COPY(4b, uint32_t)
EXPORT_COPY(8b, uint64_t)

/* 0 = general copy, 1 = batched transposition (k arrays of n x m), 2 = flat copy; the order of
 * the tests is the one of GEN_LMAD_COPY. */
int ref_lmad_classify(int r, int64_t *dst_strides, int64_t *src_strides, int64_t *shape, int64_t *knm) {
  if (lmad_map_tr(&knm[0], &knm[1], &knm[2], r, dst_strides, src_strides, shape)) return 1;
  if (lmad_memcpyable(r, dst_strides, src_strides, shape)) return 2;
  return 0;
}
