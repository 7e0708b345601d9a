// Small gflags-compatible command-line parser for the flowwalker CLI: --name=value,
// --name value, --flag, --noflag, --flag=true|false.  (gflags itself is not a dependency.)
// Flag names and defaults are those of the reference CLI (src/main.cu:40-80).
#pragma once
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <string>
#include <vector>

namespace fwflags {

struct Flag {
  enum Kind { kBool, kInt, kDouble, kString } kind;
  std::string value;  // textual value
  std::string help;
};

class Parser {
 public:
  void add(const std::string& name, Flag::Kind kind, const std::string& def, const std::string& help) {
    flags_[name] = Flag{kind, def, help};
    order_.push_back(name);
  }
  // Returns false (and fills err) on an unknown flag or a malformed value.
  bool parse(int argc, char** argv, std::string* err) {
    for (int i = 1; i < argc; ++i) {
      std::string arg = argv[i];
      if (arg == "--help" || arg == "-h") { help_ = true; continue; }
      if (arg.size() < 2 || arg[0] != '-') { *err = "unexpected argument: " + arg; return false; }
      arg = arg.substr(arg[1] == '-' ? 2 : 1);
      std::string name = arg, value;
      bool has_value = false;
      const size_t eq = arg.find('=');
      if (eq != std::string::npos) { name = arg.substr(0, eq); value = arg.substr(eq + 1); has_value = true; }
      auto it = flags_.find(name);
      if (it == flags_.end() && name.rfind("no", 0) == 0 && !has_value) {
        auto neg = flags_.find(name.substr(2));
        if (neg != flags_.end() && neg->second.kind == Flag::kBool) { neg->second.value = "false"; continue; }
      }
      if (it == flags_.end()) { *err = "unknown flag --" + name; return false; }
      Flag& f = it->second;
      if (f.kind == Flag::kBool) {
        if (!has_value) value = "true";
        if (value == "1" || value == "t" || value == "yes") value = "true";
        if (value == "0" || value == "f" || value == "no") value = "false";
        if (value != "true" && value != "false") { *err = "bad boolean for --" + name + ": " + value; return false; }
      } else {
        if (!has_value) {
          if (i + 1 >= argc) { *err = "missing value for --" + name; return false; }
          value = argv[++i];
        }
        char* end = nullptr;
        if (f.kind == Flag::kInt) { strtoll(value.c_str(), &end, 10); if (!end || *end) { *err = "bad integer for --" + name + ": " + value; return false; } }
        if (f.kind == Flag::kDouble) { strtod(value.c_str(), &end); if (!end || *end) { *err = "bad number for --" + name + ": " + value; return false; } }
      }
      f.value = value;
    }
    return true;
  }
  bool help_requested() const { return help_; }
  void print_help(const char* prog) const {
    printf("usage: %s [flags]\n", prog);
    for (const std::string& n : order_) {
      const Flag& f = flags_.at(n);
      printf("  --%-14s %s (default: %s)\n", n.c_str(), f.help.c_str(), f.value.c_str());
    }
  }
  bool b(const std::string& n) const { return flags_.at(n).value == "true"; }
  long long i(const std::string& n) const { return atoll(flags_.at(n).value.c_str()); }
  double d(const std::string& n) const { return atof(flags_.at(n).value.c_str()); }
  const std::string& s(const std::string& n) const { return flags_.at(n).value; }
  void set(const std::string& n, const std::string& v) { flags_.at(n).value = v; }

 private:
  std::map<std::string, Flag> flags_;
  std::vector<std::string> order_;
  bool help_ = false;
};

}  // namespace fwflags
