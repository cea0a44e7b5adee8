// main.cu -- appMain<SampleType, App>(argc, argv, checkResults): the command line of the
// reference's src/main.cu:5-54 (flags -g -t -f -n -c -p -k -l, long names accepted too), parsed
// without the AnyOption library.
#ifndef NEXTDOOR_B200_COMPAT_MAIN_CU
#define NEXTDOOR_B200_COMPAT_MAIN_CU
#include "nextdoor.cu"

template <class SampleType, typename App>
int appMain(int argc, char *argv[], bool (*checkResults)(NextDoorData<SampleType, App> &nextDoorData)) {
  const char *usage =
      "usage: \n\n"
      "-h --help              Prints this help\n"
      "-g --graph-file        File containing graph\n"
      "-t --graph-type <type> Format of graph file: 'adj-list' or 'edge-list'\n"
      "-f --format <format>   Format of graph file: 'binary' or 'text'\n"
      "-n --nruns             Number of runs\n"
      "-c --check-results     Check results using an algorithm\n"
      "-p --print-samples     Print Samples\n"
      "-k --kernel-type       Type of Kernel: 'SampleParallel' or 'TransitParallel'\n"
      "-l --load-balancing    Enable Load Balancing\n";
  const char *file = nullptr, *type = nullptr, *format = nullptr, *kernel = "TransitParallel";
  int nruns = 1;
  bool check = false, print = false, lb = false;
  auto is = [](const char *a, const char *s, const char *l) { return strcmp(a, s) == 0 || strcmp(a, l) == 0; };
  for (int i = 1; i < argc; i++) {
    const char *a = argv[i];
    const char *val = i + 1 < argc ? argv[i + 1] : nullptr;
    if (is(a, "-h", "--help")) { printf("%s", usage); return 0; }
    else if (is(a, "-g", "--graph-file") && val) { file = val; i++; }
    else if (is(a, "-t", "--graph-type") && val) { type = val; i++; }
    else if ((is(a, "-f", "--format") || strcmp(a, "--graph-format") == 0) && val) { format = val; i++; }
    else if (is(a, "-n", "--nruns") && val) { nruns = atoi(val); i++; }
    else if (is(a, "-k", "--kernel-type") && val) { kernel = val; i++; }
    else if (is(a, "-c", "--check-results")) check = true;
    else if (is(a, "-p", "--print-samples")) print = true;
    else if (is(a, "-l", "--load-balancing")) lb = true;
  }
  if (argc <= 1 || !file || !type || !format) { printf("%s", usage); return 0; }
  nextdoor<SampleType, App>(file, type, format, nruns, check, print, kernel, lb, checkResults);
  return 0;
}
#endif
