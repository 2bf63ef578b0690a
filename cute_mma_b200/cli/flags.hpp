// Minimal "--name value" / "--switch" parser for the two benchmark drivers (the reference uses
// p-ranav/argparse, fetched at configure time; nothing is fetched here).
#pragma once
#include <cstdlib>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

class Flags {
 public:
  // names: every accepted spelling mapped to its canonical key; switches take no value.
  void add(const std::vector<std::string>& names, const std::string& def, bool is_switch = false) {
    for (const auto& n : names) canon_[n] = names.back();
    values_[names.back()] = def;
    switch_[names.back()] = is_switch;
  }
  void parse(int argc, char** argv) {
    for (int i = 1; i < argc; ++i) {
      auto it = canon_.find(argv[i]);
      if (it == canon_.end()) throw std::runtime_error(std::string("unknown argument ") + argv[i]);
      if (switch_[it->second]) { values_[it->second] = "1"; continue; }
      if (i + 1 >= argc) throw std::runtime_error(std::string("missing value after ") + argv[i]);
      values_[it->second] = argv[++i];
    }
  }
  int geti(const std::string& k) const { return std::atoi(values_.at(k).c_str()); }
  double getd(const std::string& k) const { return std::atof(values_.at(k).c_str()); }
  bool getb(const std::string& k) const { return values_.at(k) == "1"; }
  std::string gets(const std::string& k) const { return values_.at(k); }

 private:
  std::map<std::string, std::string> canon_, values_;
  std::map<std::string, bool> switch_;
};
