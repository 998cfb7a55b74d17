// Implementation of the UPMEM host API stand-in declared in dpu.h.
// TEST INFRASTRUCTURE ONLY: lets the reference's pim_lut_host.cpp / amm_host.cpp and its DPU
// kernel run unmodified on host threads (a functional model; see dpu.h).
#include "dpu.h"

#include <dlfcn.h>
#include <unistd.h>

#include <atomic>
#include <cstring>
#include <fstream>
#include <map>
#include <string>
#include <thread>
#include <vector>

namespace {

struct Instance {  // one loaded copy of the kernel object = one DPU's worth of globals
    void* handle = nullptr;
    int (*main_fn)() = nullptr;
    void (*set_tasklet)(uint32_t) = nullptr;
    unsigned nr_tasklets = 0;
    std::map<std::string, std::pair<void*, size_t>> syms;
};

const char* kSymbols[] = {"lut_table", "input_index", "output_data", "dpu_arguments"};

}  // namespace

struct shim_set {
    uint32_t n = 0;
    std::vector<void*> prepared;                                          // per DPU: buffer of the pending transfer
    std::map<std::string, std::vector<std::vector<unsigned char>>> mram;  // symbol -> per-DPU contents
    std::vector<Instance> inst;
};

extern "C" {

uint32_t shim_count(struct dpu_set_t set) { return set.single >= 0 ? 1u : set.impl->n; }
struct dpu_set_t shim_nth(struct dpu_set_t set, uint32_t i) {
    struct dpu_set_t d = {set.impl, set.single >= 0 ? set.single : (int32_t)i};
    return d;
}

dpu_error_t dpu_alloc(uint32_t nr_dpus, const char*, struct dpu_set_t* set) {
    shim_set* s = new shim_set();
    s->n = nr_dpus;
    s->prepared.assign(nr_dpus, nullptr);
    set->impl = s;
    set->single = -1;
    return DPU_OK;
}
dpu_error_t dpu_alloc_ranks(uint32_t nr_ranks, const char* profile, struct dpu_set_t* set) {
    return dpu_alloc(nr_ranks * NR_DPUS_PER_RANK, profile, set);
}
dpu_error_t dpu_get_nr_dpus(struct dpu_set_t set, uint32_t* nr) {
    *nr = set.impl->n;
    return DPU_OK;
}

static void unload(shim_set* s) {
    for (Instance& in : s->inst)
        if (in.handle) dlclose(in.handle);
    s->inst.clear();
}

dpu_error_t dpu_load(struct dpu_set_t set, const char* path, void*) {
    shim_set* s = set.impl;
    unload(s);
    unsigned copies = std::thread::hardware_concurrency() / 4;
    if (copies < 1) copies = 1;
    if (copies > s->n) copies = s->n;
    std::ifstream src(path, std::ios::binary);
    if (!src) { fprintf(stderr, "dpu shim: cannot open kernel object %s\n", path); return DPU_ERR_SHIM; }
    const std::string bytes((std::istreambuf_iterator<char>(src)), std::istreambuf_iterator<char>());
    static std::atomic<unsigned> serial{0};
    for (unsigned k = 0; k < copies; ++k) {
        // every dlopen of a distinct file gives a private set of the kernel's globals
        const std::string tmp = "/tmp/lutamm_dpu_" + std::to_string(getpid()) + "_" + std::to_string(serial++) + ".so";
        { std::ofstream out(tmp, std::ios::binary); out.write(bytes.data(), (std::streamsize)bytes.size()); }
        Instance in;
        in.handle = dlopen(tmp.c_str(), RTLD_NOW | RTLD_LOCAL);
        unlink(tmp.c_str());
        if (!in.handle) { fprintf(stderr, "dpu shim: dlopen failed: %s\n", dlerror()); return DPU_ERR_SHIM; }
        in.main_fn = reinterpret_cast<int (*)()>(dlsym(in.handle, "dpu_main"));
        in.set_tasklet = reinterpret_cast<void (*)(uint32_t)>(dlsym(in.handle, "shim_set_tasklet"));
        const unsigned* nt = static_cast<const unsigned*>(dlsym(in.handle, "shim_nr_tasklets"));
        if (!in.main_fn || !in.set_tasklet || !nt) { fprintf(stderr, "dpu shim: %s is not a wrapped kernel\n", path); return DPU_ERR_SHIM; }
        in.nr_tasklets = *nt;
        for (const char* name : kSymbols) {
            void* p = dlsym(in.handle, name);
            const size_t* sz = static_cast<const size_t*>(dlsym(in.handle, (std::string("shim_sizeof_") + name).c_str()));
            if (p && sz) in.syms[name] = {p, *sz};
        }
        s->inst.push_back(in);
    }
    return DPU_OK;
}

dpu_error_t dpu_prepare_xfer(struct dpu_set_t dpu, void* buffer) {
    if (dpu.single < 0) return DPU_ERR_SHIM;
    dpu.impl->prepared[dpu.single] = buffer;
    return DPU_OK;
}

dpu_error_t dpu_push_xfer(struct dpu_set_t set, dpu_xfer_t xfer, const char* symbol, uint32_t offset, size_t length,
                          dpu_xfer_flags_t) {
    shim_set* s = set.impl;
    auto& per_dpu = s->mram[symbol];
    if (per_dpu.size() != s->n) per_dpu.resize(s->n);
    for (uint32_t d = 0; d < s->n; ++d) {
        void* host = s->prepared[d];
        if (!host) continue;
        std::vector<unsigned char>& m = per_dpu[d];
        if (xfer == DPU_XFER_TO_DPU) {
            if (m.size() < offset + length) m.resize(offset + length, 0);
            memcpy(m.data() + offset, host, length);
        } else {
            if (m.size() < offset + length) return DPU_ERR_SHIM;
            memcpy(host, m.data() + offset, length);
        }
    }
    return DPU_OK;
}

dpu_error_t dpu_launch(struct dpu_set_t set, dpu_launch_policy_t) {
    shim_set* s = set.impl;
    if (s->inst.empty()) return DPU_ERR_SHIM;
    std::atomic<uint32_t> next{0};
    std::atomic<int> bad{0};
    auto worker = [&](Instance* in) {
        for (uint32_t d = next++; d < s->n; d = next++) {
            for (auto& kv : in->syms) {  // this DPU's MRAM contents into the kernel's globals
                auto it = s->mram.find(kv.first);
                if (it == s->mram.end() || it->second[d].empty()) continue;
                if (it->second[d].size() > kv.second.second) { bad = 1; continue; }
                memcpy(kv.second.first, it->second[d].data(), it->second[d].size());
            }
            std::vector<std::thread> tasklets;
            for (unsigned t = 0; t < in->nr_tasklets; ++t)
                tasklets.emplace_back([in, t] { in->set_tasklet(t); in->main_fn(); });
            for (auto& th : tasklets) th.join();
            auto out = in->syms.find("output_data");
            if (out != in->syms.end()) {
                auto& per_dpu = s->mram["output_data"];
                std::vector<unsigned char>& m = per_dpu[d];
                m.resize(out->second.second);
                memcpy(m.data(), out->second.first, out->second.second);
            }
        }
    };
    s->mram["output_data"].resize(s->n);
    std::vector<std::thread> pool;
    for (Instance& in : s->inst) pool.emplace_back(worker, &in);
    for (auto& th : pool) th.join();
    return bad ? DPU_ERR_SHIM : DPU_OK;
}

dpu_error_t dpu_sync(struct dpu_set_t) { return DPU_OK; }
dpu_error_t dpu_log_read(struct dpu_set_t, FILE*) { return DPU_OK; }
dpu_error_t dpu_free(struct dpu_set_t set) {
    if (set.impl) {
        unload(set.impl);
        delete set.impl;
    }
    return DPU_OK;
}

}  // extern "C"
