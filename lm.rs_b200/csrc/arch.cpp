// arch.cpp -- registry of folder-based model architectures (arch.h)
#include "arch.h"

#include <stdio.h>
#include <sys/stat.h>

#include <map>
#include <vector>

namespace lmrs {

static std::map<std::string, ArchFactory>& registry() {
    static std::map<std::string, ArchFactory> r;
    return r;
}
void arch_register(const char* architecture, ArchFactory f) { registry()[architecture] = f; }

bool arch_is_model_dir(const std::string& path) {
    struct stat st;
    return stat(path.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}

ArchModel* arch_open(const std::string& dir, const ArchOptions& opt, std::string& err) {
    const std::string cfg_path = dir + "/config.json";
    FILE* f = fopen(cfg_path.c_str(), "rb");
    if (!f) { err = "cannot open " + cfg_path; return nullptr; }
    std::vector<char> buf;
    char tmp[4096];
    size_t n;
    while ((n = fread(tmp, 1, sizeof tmp, f)) > 0) buf.insert(buf.end(), tmp, tmp + n);
    fclose(f);
    Json cfg;
    JsonParser jp(buf.data(), buf.size());
    if (!jp.parse(cfg, err) || !cfg.is_obj()) { err = cfg_path + ": " + (err.empty() ? "not a JSON object" : err); return nullptr; }
    const std::string name = cfg.at("architecture").str;
    auto it = registry().find(name);
    if (it == registry().end()) {
        err = cfg_path + ": unknown architecture '" + name + "' (known:";
        for (const auto& kv : registry()) err += " " + kv.first;
        err += ")";
        return nullptr;
    }
    return it->second(dir, cfg, opt, err);
}

}  // namespace lmrs
