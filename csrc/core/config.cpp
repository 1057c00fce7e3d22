#include "config.hpp"
#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <fstream>
#include <sstream>

namespace dccl {

static std::string trim(const std::string& s) {
    size_t a = 0, b = s.size();
    while (a < b && std::isspace((unsigned char)s[a])) a++;
    while (b > a && std::isspace((unsigned char)s[b - 1])) b--;
    return s.substr(a, b - a);
}

static bool read_file(const std::string& path, std::string* out) {
    std::ifstream f(path);
    if (!f) return false;
    std::stringstream ss;
    ss << f.rdbuf();
    *out = ss.str();
    return true;
}

Config& Config::global() {
    static Config* c = [] { Config* x = new Config(); x->reload(); return x; }();
    return *c;
}

void Config::clear() {
    std::lock_guard<std::mutex> g(mu_);
    kv_.clear();
    file_.clear();
}

void Config::parse_ini(const std::string& text) {
    std::lock_guard<std::mutex> g(mu_);
    std::istringstream in(text);
    std::string line, section;
    while (std::getline(in, line)) {
        // strip comments (# or ;) that start a line or follow whitespace
        size_t cut = std::string::npos;
        for (size_t i = 0; i < line.size(); i++)
            if ((line[i] == '#' || line[i] == ';') && (i == 0 || std::isspace((unsigned char)line[i - 1]))) { cut = i; break; }
        if (cut != std::string::npos) line = line.substr(0, cut);
        line = trim(line);
        if (line.empty()) continue;
        if (line.front() == '[' && line.back() == ']') { section = trim(line.substr(1, line.size() - 2)); continue; }
        size_t eq = line.find('=');
        if (eq == std::string::npos) continue;
        std::string k = trim(line.substr(0, eq)), v = trim(line.substr(eq + 1));
        if (k.empty()) continue;
        kv_[section.empty() ? k : section + "/" + k] = v;
    }
}

void Config::reload() {
    clear();
    std::string text;
    const char* envf = getenv("DCCL_CONF_FILE");
    const char* candidates[] = {envf, "dccl.cfg", "derecho.cfg"};
    for (const char* c : candidates) {
        if (!c || !*c) continue;
        if (read_file(c, &text)) {
            parse_ini(text);
            std::lock_guard<std::mutex> g(mu_);
            file_ = c;
            break;
        }
    }
}

static std::string env_name_for(const std::string& key) {
    // "DCCL/allreduce_algorithm" -> "DCCL_ALLREDUCE_ALGORITHM"; only section DCCL maps to env
    if (key.compare(0, 5, "DCCL/") != 0) return "";
    std::string e = "DCCL_" + key.substr(5);
    std::transform(e.begin(), e.end(), e.begin(), [](unsigned char c) { return (char)std::toupper(c); });
    return e;
}

bool Config::has(const std::string& key) const { std::string v; return get(key, &v); }

bool Config::get(const std::string& key, std::string* out) const {
    std::string en = env_name_for(key);
    if (!en.empty()) {
        const char* e = getenv(en.c_str());
        if (e && *e) { *out = e; return true; }
    }
    std::lock_guard<std::mutex> g(mu_);
    auto it = kv_.find(key);
    if (it == kv_.end()) return false;
    *out = it->second;
    return true;
}

std::string Config::get_str(const std::string& key, const std::string& dflt) const {
    std::string v;
    return get(key, &v) ? v : dflt;
}

long long Config::get_int(const std::string& key, long long dflt) const {
    std::string v;
    if (!get(key, &v)) return dflt;
    char* end = nullptr;
    long long x = strtoll(v.c_str(), &end, 0);
    if (end == v.c_str()) return dflt;
    // size suffixes for byte-valued keys
    if (*end == 'k' || *end == 'K') x <<= 10;
    else if (*end == 'm' || *end == 'M') x <<= 20;
    else if (*end == 'g' || *end == 'G') x <<= 30;
    return x;
}

bool Config::get_bool(const std::string& key, bool dflt) const {
    std::string v;
    if (!get(key, &v)) return dflt;
    std::transform(v.begin(), v.end(), v.begin(), [](unsigned char c) { return (char)std::tolower(c); });
    if (v == "1" || v == "true" || v == "yes" || v == "on") return true;
    if (v == "0" || v == "false" || v == "no" || v == "off") return false;
    return dflt;
}

void Config::set(const std::string& key, const std::string& value) {
    std::lock_guard<std::mutex> g(mu_);
    kv_[key] = value;
}

int Config::world_size_from_layout(const std::string& json) {
    size_t p = json.find("\"min_nodes_by_shard\"");
    if (p == std::string::npos) return 0;
    p = json.find('[', p);
    if (p == std::string::npos) return 0;
    while (p < json.size() && !std::isdigit((unsigned char)json[p]) && json[p] != ']') p++;
    if (p >= json.size() || json[p] == ']') return 0;
    return atoi(json.c_str() + p);
}

static bool env_int(const char* name, int* out) {
    const char* e = getenv(name);
    if (!e || !*e) return false;
    *out = atoi(e);
    return true;
}

bool resolve_bootstrap_params(BootstrapParams* out, std::string* err) {
    BootstrapParams p;
    int rank, world, port;
    // 1. DCCL_* variables
    if (env_int("DCCL_RANK", &rank) && env_int("DCCL_WORLD_SIZE", &world)) {
        p.rank = rank; p.world = world; p.source = "env:DCCL";
        if (const char* a = getenv("DCCL_MASTER_ADDR")) p.addr = a;
        p.port = env_int("DCCL_MASTER_PORT", &port) ? port : 23580;
        *out = p;
        return true;
    }
    // 2. torchrun variables; the torch store owns MASTER_PORT, so we sit a fixed distance above it
    if (env_int("RANK", &rank) && env_int("WORLD_SIZE", &world)) {
        p.rank = rank; p.world = world; p.source = "env:torchrun";
        if (const char* a = getenv("MASTER_ADDR")) p.addr = a;
        if (env_int("DCCL_MASTER_PORT", &port)) p.port = port;
        else if (env_int("MASTER_PORT", &port)) p.port = port + 1017 > 65535 ? port - 1017 : port + 1017;
        else p.port = 23580;
        *out = p;
        return true;
    }
    // 3. configuration directory recipe
    Config& c = Config::global();
    std::string v;
    if (c.get("DERECHO/local_id", &v)) {
        p.rank = atoi(v.c_str());
        p.source = "cfg";
        if (c.get("DERECHO/contact_ip", &v) || c.get("DERECHO/leader_ip", &v)) p.addr = v;
        if (c.get("DERECHO/contact_port", &v) || c.get("DERECHO/leader_gms_port", &v)) p.port = atoi(v.c_str());
        else p.port = 23580;
        int w = (int)c.get_int("DCCL/world_size", 0);
        if (w <= 0) {
            std::string lf = c.get_str("LAYOUT/json_layout_file", "layout.json"), text;
            if (read_file(lf, &text)) w = Config::world_size_from_layout(text);
        }
        if (w <= 0) {
            if (err) *err = "configuration file gives local_id but no world size (layout.json min_nodes_by_shard or DCCL/world_size)";
            return false;
        }
        p.world = w;
        *out = p;
        return true;
    }
    // 4. nothing given: a world of one
    p.rank = 0; p.world = 1; p.port = 0; p.source = "single";
    *out = p;
    return true;
}

} // namespace dccl
