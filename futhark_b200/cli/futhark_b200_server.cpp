// The server front-end: a process that keeps one context and named variables (values that stay
// on the device) and obeys line-oriented commands on standard input -- the protocol of
// docs/server-protocol.rst, as implemented for generated programs by rts/c/server.h:323-1654.
// `futhark bench` and `futhark test` drive compiled programs through this protocol: they
// `restore` input files into variables, `call` entry points (the reply carries "runtime: N" in
// microseconds, entry point + sync), `store` results to files and `free` variables.
//
// Every reply ends with a line "%%% OK"; a failed command prints "%%% FAILURE" and the message
// before it.  Commands for sum types, arrays of records and element-wise array construction have
// no type to apply to in this library and answer with a failure.
#include <ctype.h>
#include <errno.h>
#include <getopt.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/time.h>

#include <map>
#include <string>
#include <vector>

#include "entry_table.h"

static int64_t wall_usec() {
  struct timeval t;
  gettimeofday(&t, nullptr);
  return (int64_t)t.tv_sec * 1000000 + t.tv_usec;
}

struct Server {
  futhark_context_config *cfg = nullptr;
  futhark_context *ctx = nullptr;
  std::map<std::string, fe::Value> vars;
  bool failed = false;

  void failure(const char *fmt, ...) {
    if (!failed) puts("%%% FAILURE");
    failed = true;
    va_list ap;
    va_start(ap, fmt);
    vprintf(fmt, ap);
    va_end(ap);
  }
  // reports a failed library call with the context's message
  bool bad(int rc) {
    if (rc == 0) return false;
    char *e = futhark_context_get_error(ctx);
    failure("%s\n", e ? e : "");
    free(e);
    return true;
  }
  fe::Value *var(const std::string &name) {
    auto it = vars.find(name);
    if (it == vars.end()) { failure("Unknown variable: %s\n", name.c_str()); return nullptr; }
    return &it->second;
  }
  bool fresh(const std::string &name) {
    if (vars.count(name)) { failure("Variable already exists: %s\n", name.c_str()); return false; }
    return true;
  }
  const fe::EntryPoint *entry(const std::string &name) {
    const fe::EntryPoint *e = fe::entry_point(name);
    if (e == nullptr) failure("Unknown entry point: %s\n", name.c_str());
    return e;
  }
};

// words are separated by spaces; a word in double quotes may contain spaces
static std::vector<std::string> words_of(const std::string &line) {
  std::vector<std::string> out;
  size_t i = 0;
  while (i < line.size()) {
    while (i < line.size() && isspace((unsigned char)line[i])) i++;
    if (i >= line.size()) break;
    std::string w;
    if (line[i] == '"') {
      i++;
      while (i < line.size() && line[i] != '"') w.push_back(line[i++]);
      i++;
    } else {
      while (i < line.size() && !isspace((unsigned char)line[i])) w.push_back(line[i++]);
    }
    out.push_back(w);
  }
  return out;
}

static void cmd_call(Server &s, const std::vector<std::string> &a) {
  const fe::EntryPoint *e = s.entry(a[1]);
  if (e == nullptr) return;
  if (a.size() != 3 + e->ins.size()) { s.failure("Wrong number of arguments: %s takes %d inputs.\n", e->name, (int)e->ins.size()); return; }
  std::vector<const fe::Value *> ins;
  for (size_t i = 0; i < e->ins.size(); i++) {
    fe::Value *v = s.var(a[3 + i]);
    if (v == nullptr) return;
    if (v->type != e->ins[i]) { s.failure("Wrong input type.  Expected %s, got %s.\n", e->ins[i], v->type.c_str()); return; }
    ins.push_back(v);
  }
  if (!s.fresh(a[2])) return;
  fe::Value out;
  const int64_t t0 = wall_usec();
  int rc = e->call(s.ctx, ins, out);
  rc |= futhark_context_sync(s.ctx);
  const int64_t t1 = wall_usec();
  printf("runtime: %lld\n", (long long)(t1 - t0));
  if (s.bad(rc)) { fe::release(s.ctx, out); return; }
  s.vars[a[2]] = out;
}

static void cmd_restore(Server &s, const std::vector<std::string> &a) {
  FILE *f = fopen(a[1].c_str(), "rb");
  if (f == nullptr) { s.failure("Failed to open %s: %s\n", a[1].c_str(), strerror(errno)); return; }
  int values = 0;
  bool ok = true;
  for (size_t i = 2; i + 1 < a.size() && ok; i += 2, values++) {
    const std::string &name = a[i], &type = a[i + 1];
    if (!fe::prim_type(type) && !fe::array_type(type)) { s.failure("Unknown type %s\n", type.c_str()); ok = false; break; }
    if (!s.fresh(name)) { ok = false; break; }
    std::string elem;
    int rank;
    fe::split_type(type, elem, rank);
    futhark_b200_value h;
    errno = 0;
    fe::Value v;
    if (futhark_b200_value_read(f, elem.c_str(), rank, &h) != 0) {
      s.failure("Failed to restore variable %s.\nPossibly malformed data in %s (errno: %s)\n", name.c_str(), a[1].c_str(), strerror(errno));
      ok = false;
      break;
    }
    const int rc = fe::from_host(s.ctx, type, h, v);
    // the upload reads the host buffer asynchronously: wait before it is freed
    const int rc2 = futhark_context_sync(s.ctx);
    futhark_b200_value_free(&h);
    if (s.bad(rc | rc2)) { fe::release(s.ctx, v); ok = false; break; }
    s.vars[name] = v;
  }
  if (ok && futhark_b200_value_end_of_input(f) != 0) s.failure("Expected EOF after reading %d values from %s\n", values, a[1].c_str());
  fclose(f);
}

static void cmd_store(Server &s, const std::vector<std::string> &a) {
  FILE *f = fopen(a[1].c_str(), "wb");
  if (f == nullptr) { s.failure("Failed to open %s: %s\n", a[1].c_str(), strerror(errno)); return; }
  for (size_t i = 2; i < a.size(); i++) {
    fe::Value *v = s.var(a[i]);
    if (v == nullptr) break;
    if (v->record != nullptr) { s.failure("Cannot store a value of type %s; project its fields.\n", v->type.c_str()); break; }
    futhark_b200_value h;
    int rc = fe::to_host(s.ctx, *v, h);
    rc |= futhark_context_sync(s.ctx);
    if (!s.bad(rc)) futhark_b200_value_write(f, &h, 1);       // always the binary format (rts/c/server.h: store)
    futhark_b200_value_free(&h);
    if (rc) break;
  }
  fclose(f);
}

static void dispatch(Server &s, const std::vector<std::string> &a) {
  const std::string &c = a[0];
  auto need = [&](size_t n) {
    if (a.size() < n + 1) { s.failure("Insufficient command args.\n"); return false; }
    return true;
  };
  if (c == "call") { if (need(2)) cmd_call(s, a); }
  else if (c == "restore") { if (need(1)) cmd_restore(s, a); }
  else if (c == "store") { if (need(1)) cmd_store(s, a); }
  else if (c == "free") {
    for (size_t i = 1; i < a.size(); i++) {
      fe::Value *v = s.var(a[i]);
      if (v == nullptr) return;
      s.bad(fe::release(s.ctx, *v));
      s.vars.erase(a[i]);
    }
  } else if (c == "rename") {
    if (!need(2)) return;
    fe::Value *v = s.var(a[1]);
    if (v == nullptr || !s.fresh(a[2])) return;
    s.vars[a[2]] = *v;
    s.vars.erase(a[1]);
  } else if (c == "inputs") {
    if (!need(1)) return;
    if (const fe::EntryPoint *e = s.entry(a[1]))
      for (const char *t : e->ins) puts(t);                 // no entry point consumes its arguments: no '*'
  } else if (c == "output") {
    if (!need(1)) return;
    if (const fe::EntryPoint *e = s.entry(a[1])) printf("*%s\n", e->out);   // every result is freshly allocated
  } else if (c == "clear") {
    int rc = 0;
    for (auto &kv : s.vars) rc |= fe::release(s.ctx, kv.second);
    s.vars.clear();
    rc |= futhark_context_clear_caches(s.ctx);
    s.bad(rc);
  } else if (c == "pause_profiling") { futhark_context_pause_profiling(s.ctx); }
  else if (c == "unpause_profiling") { futhark_context_unpause_profiling(s.ctx); }
  else if (c == "report") {
    char *r = futhark_context_report(s.ctx);
    if (r != nullptr) puts(r); else s.bad(1);
    free(r);
  } else if (c == "types") {
    for (const fe::PrimType &p : fe::PRIMS) puts(p.name);
    for (const fe::ArrayType &t : fe::ARRAYS) puts(t.name);
    for (const fe::RecordType &r : fe::RECORDS) puts(r.name);
  } else if (c == "entry_points") {
    for (const fe::EntryPoint &e : fe::entry_points()) puts(e.name);
  } else if (c == "kind") {
    if (!need(1)) return;
    if (fe::prim_type(a[1])) puts("primitive");
    else if (fe::array_type(a[1])) puts("array");
    else if (fe::record_type(a[1])) puts("record");
    else s.failure("Unknown type %s\n", a[1].c_str());
  } else if (c == "type") {
    if (!need(1)) return;
    if (fe::Value *v = s.var(a[1])) puts(v->type.c_str());
  } else if (c == "rank" || c == "elemtype") {
    if (!need(1)) return;
    const fe::ArrayType *t = fe::array_type(a[1]);
    if (t == nullptr) { s.failure("Not an array type\n"); return; }
    if (c == "rank") printf("%d\n", t->rank); else puts(t->elem);
  } else if (c == "shape") {
    if (!need(1)) return;
    fe::Value *v = s.var(a[1]);
    if (v == nullptr) return;
    if (v->array == nullptr) { s.failure("Not an array type\n"); return; }
    const int64_t *sh = v->array->shape(s.ctx, v->arr);
    for (int d = 0; d < v->array->rank; d++) printf("%lld\n", (long long)sh[d]);
  } else if (c == "fields") {
    if (!need(1)) return;
    const fe::RecordType *r = fe::record_type(a[1]);
    if (r == nullptr) { s.failure("Not a record type\n"); return; }
    for (size_t i = 0; i < r->fields.size(); i++) printf("%d %s\n", (int)i, r->fields[i]);
  } else if (c == "project") {
    // project TO FROM FIELD: a new reference to the field (the record stays as it is)
    if (!need(3)) return;
    fe::Value *from = s.var(a[2]);
    if (from == nullptr) return;
    if (from->record == nullptr) { s.failure("Not a record type\n"); return; }
    const size_t k = (size_t)atoi(a[3].c_str());
    if (k >= from->record->fields.size() || a[3] != std::to_string(k)) { s.failure("No such field\n"); return; }
    if (!s.fresh(a[1])) return;
    fe::Value fld;
    if (s.bad(from->record->project(s.ctx, from->arr, (int)k, fld))) return;
    s.vars[a[1]] = fld;
  } else if (c == "new") {
    // new V0 TYPE V1 ... VN: a record from variables of the field types (which stay valid)
    if (!need(2)) return;
    const fe::RecordType *r = fe::record_type(a[2]);
    if (r == nullptr) { s.failure("Not a record type\n"); return; }
    if (a.size() != 3 + r->fields.size()) { s.failure("%d fields expected but %d values provided.\n", (int)r->fields.size(), (int)a.size() - 3); return; }
    if (!s.fresh(a[1])) return;
    std::vector<const fe::Value *> fields;
    for (size_t i = 0; i < r->fields.size(); i++) {
      fe::Value *v = s.var(a[3 + i]);
      if (v == nullptr) return;
      if (v->type != r->fields[i]) { s.failure("Field %d mismatch: expected type %s, got %s\n", (int)i, r->fields[i], v->type.c_str()); return; }
      fields.push_back(v);
    }
    void *obj = nullptr;
    if (s.bad(r->make(s.ctx, fields, &obj))) return;
    fe::Value rec;
    fe::set_record(rec, r->name, obj);
    s.vars[a[1]] = rec;
  } else if (c == "set_tuning_param") {
    if (!need(2)) return;
    if (futhark_context_config_set_tuning_param(s.cfg, a[1].c_str(), (size_t)atol(a[2].c_str())) != 0)
      s.failure("Unknown tuning parameter: %s\n", a[1].c_str());
  } else if (c == "tuning_params") {
    if (!need(1)) return;
    if (s.entry(a[1]) == nullptr) return;
    for (int i = 0; i < futhark_get_tuning_param_count(); i++) printf("%s %s\n", futhark_get_tuning_param_name(i), futhark_get_tuning_param_class(i));
  } else if (c == "tuning_param_class") {
    if (!need(1)) return;
    for (int i = 0; i < futhark_get_tuning_param_count(); i++)
      if (a[1] == futhark_get_tuning_param_name(i)) { puts(futhark_get_tuning_param_class(i)); return; }
    s.failure("Unknown tuning parameter: %s\n", a[1].c_str());
  } else if (c == "attributes") {
    if (need(1)) s.entry(a[1]);                                  // no entry point has attributes
  } else if (c == "new_array" || c == "set" || c == "index" || c == "zip" || c == "unzip" || c == "variants" || c == "construct" ||
             c == "destruct" || c == "variant") {
    s.failure("Command %s does not apply to any type of this program.\n", c.c_str());
  } else {
    s.failure("Unknown command: %s\n", c.c_str());
  }
}

int main(int argc, char **argv) {
  Server s;
  s.cfg = futhark_context_config_new();
  static struct option longopts[] = {{"debugging", no_argument, nullptr, 'D'}, {"log", no_argument, nullptr, 'L'},
                                     {"profile", no_argument, nullptr, 'P'},   {"help", no_argument, nullptr, 'h'},
                                     {"print-params", no_argument, nullptr, 1}, {"param", required_argument, nullptr, 2},
                                     {"tuning", required_argument, nullptr, 3}, {"cache-file", required_argument, nullptr, 4},
                                     {"device", required_argument, nullptr, 'd'}, {nullptr, 0, nullptr, 0}};
  int ch;
  while ((ch = getopt_long(argc, argv, ":DLPhd:", longopts, nullptr)) != -1) {
    switch (ch) {
      case 'D': futhark_context_config_set_debugging(s.cfg, 1); break;
      case 'L': futhark_context_config_set_logging(s.cfg, 1); break;
      case 'P': futhark_context_config_set_profiling(s.cfg, 1); break;
      case 'd': futhark_context_config_set_device(s.cfg, optarg); break;
      case 'h': printf("Usage: %s [-D] [-L] [-P] [-d DEVICE] [--print-params] [--param NAME=VALUE] [--tuning FILE] [--cache-file FILE]\n", argv[0]); return 0;
      case 1:
        for (int i = 0; i < futhark_get_tuning_param_count(); i++) printf("%s (%s)\n", futhark_get_tuning_param_name(i), futhark_get_tuning_param_class(i));
        return 0;
      case 2: {
        char *eq = strstr(optarg, "=");
        if (eq == nullptr) { fprintf(stderr, "Invalid argument for --parameter option: %s\n", optarg); return 1; }
        *eq = 0;
        if (futhark_context_config_set_tuning_param(s.cfg, optarg, (size_t)atoi(eq + 1)) != 0) { fprintf(stderr, "Unknown tuning parameter: %s\n", optarg); return 1; }
        break;
      }
      case 3: {
        FILE *f = fopen(optarg, "r");
        if (f == nullptr) { fprintf(stderr, "When loading tuning file '%s': cannot open file\n", optarg); return 1; }
        char line[512];
        while (fgets(line, sizeof(line), f)) {
          char *eq = strstr(line, "=");
          if (eq == nullptr) continue;
          *eq = 0;
          futhark_context_config_set_tuning_param(s.cfg, line, (size_t)atoi(eq + 1));
        }
        fclose(f);
        break;
      }
      case 4: futhark_context_config_set_cache_file(s.cfg, optarg); break;
      default: fprintf(stderr, "Unknown or incomplete option: %s\n", argv[optind - 1]); return 1;
    }
  }
  s.ctx = futhark_context_new(s.cfg);
  {
    char *err = futhark_context_get_error(s.ctx);
    if (err != nullptr) { fprintf(stderr, "Error during context initialisation:\n%s", err); return 1; }
  }
  puts("%%% OK");                                  // initialisation has finished
  fflush(stdout);

  std::string line;
  int c;
  for (;;) {
    line.clear();
    while ((c = getchar()) != EOF && c != '\n') line.push_back((char)c);
    if (c == EOF && line.empty()) break;
    const std::vector<std::string> a = words_of(line);
    s.failed = false;
    if (!a.empty()) dispatch(s, a);
    puts("%%% OK");
    fflush(stdout);
    if (c == EOF) break;
  }
  for (auto &kv : s.vars) fe::release(s.ctx, kv.second);
  futhark_context_free(s.ctx);
  futhark_context_config_free(s.cfg);
  return 0;
}
