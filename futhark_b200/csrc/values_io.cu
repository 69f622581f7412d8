// Host-side value input/output in the two formats of the reference's compiled executables:
// the textual Futhark value syntax and the binary data format
// (docs/binary-data-format.rst; behaviour of rts/c/values.h:18-845).  With it, the data files
// that `futhark dataset`, `futhark test` and `futhark bench` produce and consume can drive this
// library's entry points (futhark_b200/cli/futhark_b200_cli.cpp is the executable front-end).
//
// Pure host code (no kernels); it lives in the shared library so that any host language can use
// it through the C ABI.  Readers are typed, as the reference's are: the caller states the element
// type and rank it expects (an entry point's signature), text elements may carry the type suffix
// or omit it, and a binary value whose header disagrees is an error.  Errors are returned (code
// 1, message from futhark_b200_value_error) rather than ending the process.
#include <cuda_fp16.h>
#include <ctype.h>
#include <errno.h>
#include <inttypes.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include "../../include/futhark_b200.h"

namespace {

thread_local std::string g_error;

int fail(const std::string &msg) {
  g_error = msg;
  return 1;
}

enum Kind { K_SINT, K_UINT, K_F16, K_F32, K_F64, K_BOOL };
struct Prim {
  const char *name;      // "i32"
  const char *binname;   // " i32": right-aligned in four characters
  int size;
  Kind kind;
};
const Prim PRIMS[] = {
    {"i8", "  i8", 1, K_SINT},  {"i16", " i16", 2, K_SINT}, {"i32", " i32", 4, K_SINT}, {"i64", " i64", 8, K_SINT},
    {"u8", "  u8", 1, K_UINT},  {"u16", " u16", 2, K_UINT}, {"u32", " u32", 4, K_UINT}, {"u64", " u64", 8, K_UINT},
    {"f16", " f16", 2, K_F16},  {"f32", " f32", 4, K_F32},  {"f64", " f64", 8, K_F64},  {"bool", "bool", 1, K_BOOL},
};

const Prim *prim_by_name(const char *name) {
  for (const Prim &p : PRIMS)
    if (strcmp(p.name, name) == 0) return &p;
  return nullptr;
}
const Prim *prim_by_binname(const char *four) {
  for (const Prim &p : PRIMS)
    if (memcmp(p.binname, four, 4) == 0) return &p;
  return nullptr;
}

// ---- tokens of the textual syntax: runs of [A-Za-z0-9.+-_], or one other character; `--` starts
// a comment that runs to the end of the line (rts/c/values.h:29-68)
bool is_constituent(int c) { return isalnum(c) || c == '.' || c == '-' || c == '+' || c == '_'; }

void skip_blank(FILE *f) {
  int c;
  do c = getc(f);
  while (isspace(c));
  if (c != EOF) ungetc(c, f);
}

// empty string only at the end of the input
std::string next_token(FILE *f) {
  for (;;) {
    skip_blank(f);
    std::string tok;
    bool comment = false;
    for (;;) {
      const int c = getc(f);
      if (c == EOF) return tok;
      if (c == '-' && tok == "-") { comment = true; break; }
      if (!is_constituent(c)) {
        if (tok.empty()) tok.push_back((char)c);
        else ungetc(c, f);
        return tok;
      }
      tok.push_back((char)c);
    }
    if (comment) {
      int c;
      do c = getc(f);
      while (c != '\n' && c != EOF);
    }
  }
}

// ---- one scalar of the textual syntax into `dst` (prim->size bytes)
bool parse_scalar(const Prim *p, std::string tok, void *dst) {
  if (p->kind == K_BOOL) {
    if (tok == "true") { *(uint8_t *)dst = 1; return true; }
    if (tok == "false") { *(uint8_t *)dst = 0; return true; }
    return false;
  }
  std::string t;
  for (char c : tok)
    if (c != '_') t.push_back(c);
  const std::string pre = p->name;
  if (p->kind == K_F16 || p->kind == K_F32 || p->kind == K_F64) {
    double v;
    if (t == pre + ".nan") v = NAN;
    else if (t == pre + ".inf") v = INFINITY;
    else if (t == "-" + pre + ".inf") v = -INFINITY;
    else {
      char *end = nullptr;
      v = (p->kind == K_F64) ? strtod(t.c_str(), &end) : (double)strtof(t.c_str(), &end);
      if (end == t.c_str()) return false;
      if (*end != 0 && pre != end) return false;         // nothing, or exactly the type's suffix
    }
    if (p->kind == K_F64) *(double *)dst = v;
    else if (p->kind == K_F32) *(float *)dst = (float)v;
    else *(uint16_t *)dst = __half_as_ushort(__float2half_rn((float)v));
    return true;
  }
  // integers: decimal, 0x.., 0.. as scanf's %i reads them; the value wraps to the type's width
  char *end = nullptr;
  errno = 0;
  unsigned long long bits;
  if (p->kind == K_UINT && p->size == 8) bits = strtoull(t.c_str(), &end, 0);
  else bits = (unsigned long long)strtoll(t.c_str(), &end, 0);
  if (end == t.c_str()) return false;
  if (*end != 0 && pre != end) return false;
  memcpy(dst, &bits, (size_t)p->size);                   // little endian host
  return true;
}

void print_scalar(FILE *f, const Prim *p, const void *src) {
  switch (p->kind) {
    case K_SINT: {
      int64_t v = p->size == 1 ? *(const int8_t *)src : p->size == 2 ? *(const int16_t *)src : p->size == 4 ? *(const int32_t *)src : *(const int64_t *)src;
      fprintf(f, "%" PRId64 "%s", v, p->name);
      break;
    }
    case K_UINT: {
      uint64_t v = p->size == 1 ? *(const uint8_t *)src : p->size == 2 ? *(const uint16_t *)src : p->size == 4 ? *(const uint32_t *)src : *(const uint64_t *)src;
      fprintf(f, "%" PRIu64 "%s", v, p->name);
      break;
    }
    case K_BOOL: fputs(*(const uint8_t *)src ? "true" : "false", f); break;
    default: {
      double v = p->kind == K_F64 ? *(const double *)src : p->kind == K_F32 ? (double)*(const float *)src
                                                                           : (double)__half2float(__ushort_as_half(*(const uint16_t *)src));
      if (isnan(v)) fprintf(f, "%s.nan", p->name);
      else if (isinf(v)) fprintf(f, "%s%s.inf", v < 0 ? "-" : "", p->name);
      else fprintf(f, "%.*g%s", p->kind == K_F64 ? 17 : 9, v, p->name);      // digits that round-trip
    }
  }
}

// ---- textual arrays: brackets nested `rank` deep with the same extent at every level (a comma
// before a closing bracket is tolerated, as by the reference); or empty([d0]..[dk]type)
struct TextArray {
  FILE *f;
  const Prim *p;
  int rank;
  int64_t shape[8];
  bool known[8];
  std::vector<unsigned char> data;

  // the '[' of this level has been consumed
  bool level(int d) {
    int64_t count = 0;
    bool want_elem = true;
    for (;;) {
      const std::string tok = next_token(f);
      if (tok.empty()) return false;
      if (tok == "]") break;
      if (tok == ",") {
        if (want_elem) return false;
        want_elem = true;
        continue;
      }
      if (!want_elem) return false;
      if (d == rank - 1) {
        const size_t at = data.size();
        data.resize(at + (size_t)p->size);
        if (!parse_scalar(p, tok, data.data() + at)) return false;
      } else {
        if (tok != "[" || !level(d + 1)) return false;
      }
      count++;
      want_elem = false;
    }
    if (known[d]) return shape[d] == count;
    known[d] = true;
    shape[d] = count;
    return true;
  }

  bool empty_form() {                                    // after the token "empty"
    if (next_token(f) != "(") return false;
    bool any_zero = false;
    for (int d = 0; d < rank; d++) {
      if (next_token(f) != "[") return false;
      const std::string n = next_token(f);
      char *end = nullptr;
      shape[d] = (int64_t)strtoull(n.c_str(), &end, 10);
      if (end == n.c_str() || *end != 0) return false;
      if (next_token(f) != "]") return false;
      any_zero = any_zero || shape[d] == 0;
    }
    if (next_token(f) != p->name) return false;
    if (next_token(f) != ")") return false;
    return any_zero;
  }

  bool parse() {
    for (int d = 0; d < 8; d++) { shape[d] = 0; known[d] = false; }
    std::string tok = next_token(f);
    if (tok == "empty") return empty_form();
    return tok == "[" && level(0);
  }
};

int read_binary(FILE *f, const Prim *p, int rank, futhark_b200_value *out) {
  const int version = getc(f);
  if (version == EOF) return fail("binary-input: could not read version.");
  if (version != 2) return fail("binary-input: File uses version " + std::to_string(version) + ", but I only understand version 2.");
  const int dims = getc(f);
  if (dims == EOF) return fail("binary-input: Couldn't get dims.");
  char tname[4];
  if (fread(tname, 1, 4, f) != 4) return fail("binary-input: Couldn't read element type.");
  const Prim *got = prim_by_binname(tname);
  if (got == nullptr) return fail("binary-input: Did not recognize the type '" + std::string(tname, 4) + "'.");
  if (dims != rank || got != p)
    return fail("binary-input: Expected " + std::to_string(rank) + "D-array with element type '" + p->name + "' but got " +
                std::to_string(dims) + "D-array with element type '" + got->name + "'.");
  int64_t count = 1;
  for (int d = 0; d < rank; d++) {
    uint64_t ext;
    if (fread(&ext, 8, 1, f) != 1) return fail("binary-input: Couldn't read size for dimension " + std::to_string(d) + " of array.");
    out->shape[d] = (int64_t)ext;
    if (out->shape[d] < 0) return fail("binary-input: negative dimension.");
    count *= out->shape[d];
  }
  const size_t bytes = (size_t)count * (size_t)p->size;
  out->data = malloc(bytes ? bytes : 1);
  if (out->data == nullptr) return fail("binary-input: Failed to allocate array of size " + std::to_string(bytes) + ".");
  const size_t got_elems = fread(out->data, (size_t)p->size, (size_t)count, f);
  if ((int64_t)got_elems != count) {
    free(out->data);
    out->data = nullptr;
    return fail("binary-input: tried to read " + std::to_string(count) + " elements of an array, but only got " + std::to_string(got_elems) + " elements.");
  }
  return 0;
}

void write_text(FILE *f, const Prim *p, const unsigned char *data, const int64_t *shape, int rank) {
  if (rank == 0) { print_scalar(f, p, data); return; }
  int64_t slice = 1;
  for (int d = 1; d < rank; d++) slice *= shape[d];
  if (shape[0] * slice == 0) {
    fputs("empty(", f);
    for (int d = 0; d < rank; d++) fprintf(f, "[%" PRId64 "]", shape[d]);
    fprintf(f, "%s)", p->name);
    return;
  }
  fputc('[', f);
  for (int64_t i = 0; i < shape[0]; i++) {
    if (i) fputs(", ", f);
    write_text(f, p, data + i * slice * p->size, shape + 1, rank - 1);
  }
  fputc(']', f);
}

}  // namespace

extern "C" {

const char *futhark_b200_value_error(void) { return g_error.c_str(); }

int futhark_b200_value_read(FILE *f, const char *type, int rank, struct futhark_b200_value *out) {
  const Prim *p = prim_by_name(type);
  if (p == nullptr) return fail(std::string("unknown element type '") + type + "'");
  if (rank < 0 || rank > 8) return fail("rank must be 0..8");
  memset(out, 0, sizeof(*out));
  snprintf(out->type, sizeof(out->type), "%s", p->name);
  out->rank = rank;
  skip_blank(f);
  const int c = getc(f);
  if (c == 'b') return read_binary(f, p, rank, out);
  if (c != EOF) ungetc(c, f);
  if (rank == 0) {
    const std::string tok = next_token(f);
    out->data = malloc(8);
    if (tok.empty() || !parse_scalar(p, tok, out->data)) {
      free(out->data);
      out->data = nullptr;
      return fail(std::string("could not read a value of type ") + p->name);
    }
    return 0;
  }
  TextArray ta;
  ta.f = f; ta.p = p; ta.rank = rank;
  if (!ta.parse()) return fail("could not read a " + std::to_string(rank) + "-dimensional array of " + p->name);
  int64_t count = 1;
  for (int d = 0; d < rank; d++) { out->shape[d] = ta.shape[d]; count *= ta.shape[d]; }
  if ((size_t)count * (size_t)p->size != ta.data.size()) return fail("irregular array");
  out->data = malloc(ta.data.size() ? ta.data.size() : 1);
  if (out->data == nullptr) return fail("out of memory");
  memcpy(out->data, ta.data.data(), ta.data.size());
  return 0;
}

int futhark_b200_value_write(FILE *f, const struct futhark_b200_value *v, int binary) {
  const Prim *p = prim_by_name(v->type);
  if (p == nullptr) return fail(std::string("unknown element type '") + v->type + "'");
  if (v->rank < 0 || v->rank > 8) return fail("rank must be 0..8");
  if (!binary) {
    write_text(f, p, (const unsigned char *)v->data, v->shape, v->rank);
    return ferror(f) ? fail("write error") : 0;
  }
  int64_t count = 1;
  for (int d = 0; d < v->rank; d++) count *= v->shape[d];
  fputc('b', f);
  fputc(2, f);
  fputc(v->rank, f);
  fwrite(p->binname, 1, 4, f);
  fwrite(v->shape, 8, (size_t)v->rank, f);
  fwrite(v->data, (size_t)p->size, (size_t)count, f);
  return ferror(f) ? fail("write error") : 0;
}

void futhark_b200_value_free(struct futhark_b200_value *v) {
  free(v->data);
  v->data = nullptr;
}

int futhark_b200_value_end_of_input(FILE *f) { return next_token(f).empty() ? 0 : 1; }

int futhark_b200_value_read_mem(const void *buf, size_t len, size_t *consumed, const char *type, int rank,
                                struct futhark_b200_value *out) {
  if (len == 0) return fail("empty input");
  FILE *f = fmemopen(const_cast<void *>(buf), len, "rb");
  if (f == nullptr) return fail("fmemopen failed");
  const int rc = futhark_b200_value_read(f, type, rank, out);
  if (consumed != nullptr) *consumed = (size_t)ftell(f);
  fclose(f);
  return rc;
}

int futhark_b200_value_write_mem(const struct futhark_b200_value *v, int binary, void **buf, size_t *len) {
  char *mem = nullptr;
  size_t n = 0;
  FILE *f = open_memstream(&mem, &n);
  if (f == nullptr) return fail("open_memstream failed");
  const int rc = futhark_b200_value_write(f, v, binary);
  fclose(f);
  if (rc != 0) { free(mem); return rc; }
  *buf = mem;
  *len = n;
  return 0;
}

}  // extern "C"
