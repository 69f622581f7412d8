// The executable front-end: what `futhark cuda` (without --library) wraps around a program's
// entry points, for the entry points of libfuthark_b200.so.  It follows the generated main() of
// src/Futhark/CodeGen/Backends/GenericC/CLI.hs:28-470: the same options, input values read from
// standard input (text or binary, one per parameter, then end of input), an optional warm-up run
// and `-r` timed runs with the wall time of each (entry point + sync, in microseconds) written
// to the `-t` file, and the result of the last run printed to standard output in text or (`-b`)
// binary form, one value per line.  `futhark test` and `futhark bench` drive compiled programs
// through exactly this interface.
//
// Plain C++ on the library's C ABI; no CUDA code here.
#include <errno.h>
#include <getopt.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/time.h>

#include <string>
#include <vector>

#include "entry_table.h"

static void panic(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vfprintf(stderr, fmt, ap);
  va_end(ap);
  exit(code);
}

static int64_t wall_usec() {
  struct timeval t;
  gettimeofday(&t, nullptr);
  return (int64_t)t.tv_sec * 1000000 + t.tv_usec;
}

static void check(futhark_context *ctx, int rc) {
  if (rc != 0) {
    char *e = futhark_context_get_error(ctx);
    panic(1, "%s", e ? e : "unknown error\n");
  }
}

static const char *USAGE =
    "  -t/--write-runtime-to FILE Print the time taken to execute the program to the indicated file, an integral number of microseconds.\n"
    "  -r/--runs INT              Perform NUM runs of the program.\n"
    "  -D/--debugging             Perform possibly expensive internal correctness checks and verbose logging.\n"
    "  -L/--log                   Print various low-overhead logging information to stderr while running.\n"
    "  -P/--profile               Enable the collection of profiling information.\n"
    "  -e/--entry-point NAME      The entry point to run.\n"
    "  -b/--binary-output         Print the program result in the binary output format.\n"
    "  -n/--no-print-result       Do not print the program result.\n"
    "  -h/--help                  Print help information and exit.\n"
    "  --print-params             Print all tuning parameters that can be set with --param or --tuning.\n"
    "  --param ASSIGNMENT         Set a tuning parameter to the given value.\n"
    "  --tuning FILE              Read size=value assignments from the given file.\n"
    "  --cache-file FILE          Store program cache here.\n"
    "  -d/--device NAME           Use the first device whose name contains the given string.\n"
    "  --list-entry-points        Print the entry points with their parameter and result types and exit.\n";

int main(int argc, char **argv) {
  futhark_context_config *cfg = futhark_context_config_new();
  const char *entry_point = "main";
  const char *runtime_path = nullptr;
  int num_runs = 1, perform_warmup = 0, binary_output = 0, print_result = 1, profile = 0;
  static struct option longopts[] = {
      {"write-runtime-to", required_argument, nullptr, 't'}, {"runs", required_argument, nullptr, 'r'},
      {"debugging", no_argument, nullptr, 'D'},              {"log", no_argument, nullptr, 'L'},
      {"profile", no_argument, nullptr, 'P'},                {"entry-point", required_argument, nullptr, 'e'},
      {"binary-output", no_argument, nullptr, 'b'},          {"no-print-result", no_argument, nullptr, 'n'},
      {"help", no_argument, nullptr, 'h'},                   {"print-params", no_argument, nullptr, 1},
      {"param", required_argument, nullptr, 2},              {"tuning", required_argument, nullptr, 3},
      {"cache-file", required_argument, nullptr, 4},         {"device", required_argument, nullptr, 'd'},
      {"list-entry-points", no_argument, nullptr, 5},        {nullptr, 0, nullptr, 0}};
  int ch;
  while ((ch = getopt_long(argc, argv, ":t:r:DLPe:bnhd:", longopts, nullptr)) != -1) {
    switch (ch) {
      case 't': runtime_path = optarg; break;
      case 'r':
        num_runs = atoi(optarg);
        perform_warmup = 1;
        if (num_runs <= 0) panic(1, "Need a positive number of runs, not %s\n", optarg);
        break;
      case 'D': futhark_context_config_set_debugging(cfg, 1); break;
      case 'L': futhark_context_config_set_logging(cfg, 1); break;
      case 'P': futhark_context_config_set_profiling(cfg, 1); profile = 1; break;
      case 'e': entry_point = optarg; break;
      case 'b': binary_output = 1; break;
      case 'n': print_result = 0; break;
      case 'd': futhark_context_config_set_device(cfg, optarg); break;
      case 'h': printf("Usage: %s [OPTION]...\nOptions:\n\n%s\nFor more information, consult the Futhark User's Guide or the man pages.\n", argv[0], USAGE); return 0;
      case 1:
        for (int i = 0; i < futhark_get_tuning_param_count(); i++) printf("%s (%s)\n", futhark_get_tuning_param_name(i), futhark_get_tuning_param_class(i));
        return 0;
      case 2: {
        char *eq = strstr(optarg, "=");
        if (eq == nullptr) panic(1, "Invalid argument for --parameter option: %s\n", optarg);
        *eq = 0;
        if (futhark_context_config_set_tuning_param(cfg, optarg, (size_t)atoi(eq + 1)) != 0) panic(1, "Unknown tuning parameter: %s\n", optarg);
        break;
      }
      case 3: {  // lines of name=value (rts/c/tuning.h)
        FILE *f = fopen(optarg, "r");
        if (f == nullptr) panic(1, "When loading tuning file '%s': cannot open file\n", optarg);
        char line[512];
        while (fgets(line, sizeof(line), f)) {
          char *eq = strstr(line, "=");
          if (eq == nullptr) continue;
          *eq = 0;
          if (futhark_context_config_set_tuning_param(cfg, line, (size_t)atoi(eq + 1)) != 0)
            panic(1, "When loading tuning file '%s': Unknown name '%s'\n", optarg, line);
        }
        fclose(f);
        break;
      }
      case 4: futhark_context_config_set_cache_file(cfg, optarg); break;
      case 5:
        for (const fe::EntryPoint &e : fe::entry_points()) {
          printf("%s:", e.name);
          for (const char *t : e.ins) printf(" %s", t);
          printf(" -> %s\n", e.out);
        }
        return 0;
      case ':': panic(-1, "Missing argument for option %s\n", argv[optind - 1]);
      default: panic(-1, "Unknown option: %s\n", argv[optind - 1]);
    }
  }
  if (optind != argc) panic(1, "Excess non-option: %s\n", argv[optind]);

  const fe::EntryPoint *entry = fe::entry_point(entry_point);
  if (entry == nullptr) {
    fprintf(stderr, "No entry point '%s'.  Select another with --entry-point.  Options are:\n", entry_point);
    for (const fe::EntryPoint &e : fe::entry_points()) fprintf(stderr, "%s\n", e.name);
    return 1;
  }

  FILE *runtime_file = nullptr;
  if (runtime_path != nullptr) {
    runtime_file = fopen(runtime_path, "w");
    if (runtime_file == nullptr) panic(1, "Cannot open %s: %s\n", runtime_path, strerror(errno));
  }

  futhark_context *ctx = futhark_context_new(cfg);
  {
    char *err = futhark_context_get_error(ctx);
    if (err != nullptr) panic(1, "Error during context initialisation:\n%s", err);
  }
  futhark_context_pause_profiling(ctx);       // initialisation is not profiled (CLI.hs:385-386)

  // read the arguments, then insist on the end of the input (CLI.hs:388-394)
  std::vector<futhark_b200_value> parsed(entry->ins.size());
  for (size_t i = 0; i < entry->ins.size(); i++) {
    std::string elem;
    int rank;
    fe::split_type(entry->ins[i], elem, rank);
    if (futhark_b200_value_read(stdin, elem.c_str(), rank, &parsed[i]) != 0)
      panic(1, "Error when reading input #%d of type %s (errno: %s).\n%s\n", (int)i, entry->ins[i], strerror(errno), futhark_b200_value_error());
  }
  if (futhark_b200_value_end_of_input(stdin) != 0) panic(1, "Expected EOF on stdin after reading input for \"%s\".\n", entry->name);

  fe::Value result;
  auto run_once = [&](bool timed, bool profiled) {
    // the arguments are packed into fresh arrays for every run, outside the timed region
    std::vector<fe::Value> args(entry->ins.size());
    std::vector<const fe::Value *> argp;
    for (size_t i = 0; i < args.size(); i++) {
      if (fe::from_host(ctx, entry->ins[i], parsed[i], args[i]) != 0) check(ctx, 1);
      argp.push_back(&args[i]);
    }
    check(ctx, futhark_context_sync(ctx));
    if (profiled) futhark_context_unpause_profiling(ctx);
    const int64_t t0 = wall_usec();
    check(ctx, entry->call(ctx, argp, result));
    check(ctx, futhark_context_sync(ctx));
    if (profiled) futhark_context_pause_profiling(ctx);
    const int64_t t1 = wall_usec();
    if (timed && runtime_file != nullptr) {
      fprintf(runtime_file, "%lld\n", (long long)(t1 - t0));
      fflush(runtime_file);
    }
    for (fe::Value &a : args) check(ctx, fe::release(ctx, a));
  };
  if (perform_warmup) {
    run_once(false, false);
    check(ctx, fe::release(ctx, result));
  }
  for (int run = 0; run < num_runs; run++) {
    run_once(true, run == num_runs - 1);       // only the last run is profiled
    if (run < num_runs - 1) check(ctx, fe::release(ctx, result));
  }
  for (futhark_b200_value &v : parsed) futhark_b200_value_free(&v);

  if (print_result) {
    // a tuple's fields are projected and printed one per line (CLI.hs:279-296)
    std::vector<fe::Value> outs;
    if (result.record == nullptr) outs.push_back(result);
    else
      for (size_t k = 0; k < result.record->fields.size(); k++) {
        fe::Value f;
        check(ctx, result.record->project(ctx, result.arr, (int)k, f));
        outs.push_back(f);
      }
    for (fe::Value &v : outs) {
      futhark_b200_value h;
      check(ctx, fe::to_host(ctx, v, h));
      check(ctx, futhark_context_sync(ctx));
      futhark_b200_value_write(stdout, &h, binary_output);
      puts("");
      futhark_b200_value_free(&h);
      if (result.record != nullptr) check(ctx, fe::release(ctx, v));
    }
  }
  check(ctx, fe::release(ctx, result));
  if (runtime_file != nullptr) fclose(runtime_file);
  if (profile) {
    char *report = futhark_context_report(ctx);
    fputs(report, stderr);
    free(report);
  }
  futhark_context_free(ctx);
  futhark_context_config_free(cfg);
  return 0;
}
