/**
 * Configuration: environment > configuration file > built-in default.
 *
 * The file is an INI file in the working directory, spelled like the
 * derecho.cfg the original reads through Derecho's Conf (reference
 * src/application/cfg/n0/derecho.cfg; keys looked up as "SECTION/key",
 * reference dccl.cpp:412-413). Searched in this order: $DCCL_CONF_FILE,
 * ./dccl.cfg, ./derecho.cfg. The world size of the cfg-directory recipe comes
 * from the layout file named by LAYOUT/json_layout_file (min_nodes_by_shard).
 *
 * A key SECTION/key of section DCCL can also be given as the environment
 * variable DCCL_<KEY> (upper case), e.g. DCCL_ALLREDUCE_ALGORITHM=ring.
 */
#pragma once
#include <map>
#include <mutex>
#include <string>

namespace dccl {

class Config {
public:
    /** Process-wide instance, loaded from the working directory on first use. */
    static Config& global();
    /** Re-read files and environment (tests change directory between runs). */
    void reload();
    /** Parse INI text; used by reload() and directly by unit tests. */
    void parse_ini(const std::string& text);
    void clear();

    bool has(const std::string& key) const;
    /** Lookup with environment override; false when absent everywhere. */
    bool get(const std::string& key, std::string* out) const;
    std::string get_str(const std::string& key, const std::string& dflt) const;
    long long get_int(const std::string& key, long long dflt) const;
    bool get_bool(const std::string& key, bool dflt) const;
    void set(const std::string& key, const std::string& value);
    const std::string& loaded_file() const { return file_; }

    /** World size from a layout.json text: first number in "min_nodes_by_shard"; 0 when absent. */
    static int world_size_from_layout(const std::string& json_text);

private:
    std::map<std::string, std::string> kv_;
    std::string file_;
    mutable std::mutex mu_;
};

/** Rank / world / rendezvous address resolved from env or files. */
struct BootstrapParams {
    int rank = -1;
    int world = -1;
    std::string addr = "127.0.0.1";
    int port = 0;
    std::string source;  // "env:DCCL", "env:torchrun", "cfg", "single"
};
bool resolve_bootstrap_params(BootstrapParams* out, std::string* err);

} // namespace dccl
