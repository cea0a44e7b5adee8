// Stand-in for the third-party AnyOption header that the reference's src/main.cu includes and
// that is not part of the reference tree.  Only lets appMain() compile; ref_gpu.cu never calls it.
#pragma once
class AnyOption {
 public:
  void addUsage(const char *) {}
  void setFlag(const char *, char) {}
  void setOption(const char *, char) {}
  void processCommandArgs(int, char **) {}
  bool hasOptions() { return false; }
  void printUsage() {}
  char *getValue(char) { return nullptr; }
  char *getValue(const char *) { return nullptr; }
  bool getFlag(char) { return false; }
  bool getFlag(const char *) { return false; }
};
