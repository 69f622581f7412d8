/* Thin exports of the reference's OWN value reader/writer (rts/c/values.h), compiled from the
 * header where it lies in the reference checkout (never copied into this repository).
 * TEST INFRASTRUCTURE ONLY: the tests of this library's value input/output read what the
 * reference writes and let the reference read what this library writes, in both formats.
 *
 * Built by oracle/build.py into oracle/_ref/libref_values.so when the reference checkout is
 * present; its rts/c directory is given with -I.  The header expects the runtime's panic
 * function and the half-precision conversions; the former is supplied here (tests feed the
 * reference well-formed input only), the latter come from the reference's half.h.
 */
#define _GNU_SOURCE
#include <assert.h>
#include <ctype.h>
#include <errno.h>
#include <float.h>
#include <inttypes.h>
#include <math.h>
#include <stdarg.h>
#include <stdbool.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static void futhark_panic(int eval, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vfprintf(stderr, fmt, ap);
  va_end(ap);
  exit(eval);
}

#define SCALAR_FUN_ATTR static inline
#include "half.h"
#include "values.h"

static const struct primtype_info_t *by_name(const char *name) {
  for (const struct primtype_info_t **t = primtypes; *t != NULL; t++)
    if (strcmp((*t)->type_name, name) == 0) return *t;
  return NULL;
}

/* writes one value (rank 0 = scalar) into a malloc'd buffer */
int ref_write_value(const char *type, int binary, const void *data, const int64_t *shape, int rank, char **out, size_t *len) {
  const struct primtype_info_t *t = by_name(type);
  if (t == NULL) return 2;
  FILE *f = open_memstream(out, len);
  int rc = rank == 0 ? write_scalar(f, binary, t, (void *)data) < 0 : write_array(f, binary, t, data, shape, (int8_t)rank);
  fclose(f);
  return rc;
}

/* reads one value; *data is malloc'd; returns the reference's status (0 = ok) */
int ref_read_value(const char *type, const void *buf, size_t len, void **data, int64_t *shape, int rank) {
  const struct primtype_info_t *t = by_name(type);
  if (t == NULL) return 2;
  FILE *f = fmemopen((void *)buf, len, "rb");
  int rc;
  *data = NULL;
  if (rank == 0) {
    *data = malloc(8);
    rc = read_scalar(f, t, *data);
  } else {
    rc = read_array(f, t, data, shape, rank);
  }
  if (rc == 0) rc = end_of_input(f) ? 3 : 0;
  fclose(f);
  return rc;
}

void ref_free(void *p) { free(p); }
