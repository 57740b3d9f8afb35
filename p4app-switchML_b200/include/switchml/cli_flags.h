// Tiny "--name value" / "--name=value" command line reader shared by the example and
// benchmark programs (the reference uses boost::program_options for the same purpose).
#ifndef SWITCHML_CLI_FLAGS_H_
#define SWITCHML_CLI_FLAGS_H_

#include <cstdlib>
#include <iostream>
#include <map>
#include <string>
#include <vector>

namespace switchml {

class CliFlags {
 public:
  // Declare a flag with its default and help text; returns *this for chaining.
  CliFlags& Add(const std::string& name, const std::string& def, const std::string& help) {
    order_.push_back(name);
    values_[name] = def;
    help_[name] = help;
    return *this;
  }
  // False on --help or on an unknown flag (after printing the usage).
  bool Parse(int argc, char** argv, const std::string& title) {
    for (int i = 1; i < argc; i++) {
      std::string a = argv[i];
      if (a == "-h" || a == "--help") { Usage(title); return false; }
      if (a.rfind("--", 0) != 0) { std::cerr << "unexpected argument '" << a << "'\n"; Usage(title); return false; }
      std::string name = a.substr(2), value;
      size_t eq = name.find('=');
      if (eq != std::string::npos) {
        value = name.substr(eq + 1);
        name = name.substr(0, eq);
      } else if (i + 1 < argc) {
        value = argv[++i];
      } else {
        std::cerr << "flag --" << name << " needs a value\n";
        return false;
      }
      if (!values_.count(name)) { std::cerr << "unknown flag --" << name << "\n"; Usage(title); return false; }
      values_[name] = value;
    }
    return true;
  }
  std::string Str(const std::string& n) const { return values_.at(n); }
  uint64_t U64(const std::string& n) const { return strtoull(values_.at(n).c_str(), nullptr, 0); }
  double F64(const std::string& n) const { return strtod(values_.at(n).c_str(), nullptr); }
  bool Bool(const std::string& n) const {
    const std::string& v = values_.at(n);
    return v == "1" || v == "true" || v == "yes" || v == "on";
  }
  void Usage(const std::string& title) const {
    std::cout << title << "\n";
    for (const std::string& n : order_)
      std::cout << "  --" << n << " (default: " << values_.at(n) << ")\n      " << help_.at(n) << "\n";
  }

 private:
  std::vector<std::string> order_;
  std::map<std::string, std::string> values_, help_;
};

}  // namespace switchml
#endif  // SWITCHML_CLI_FLAGS_H_
