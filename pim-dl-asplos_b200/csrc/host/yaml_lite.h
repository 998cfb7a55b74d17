// Minimal reader/writer for the configuration files of the inference engine: a YAML subset
// of two-level maps of scalars ("section:" then indented "key: value"), '#' comments and
// optional quotes.  That is all the reference's configs/*.yaml use; its own parser is
// yaml-cpp, which is not part of this library.
#pragma once
#include <fstream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

namespace yaml_lite {

struct Doc {
    // section -> ordered (key, value)
    std::vector<std::pair<std::string, std::vector<std::pair<std::string, std::string>>>> sections;

    const std::string* find(const std::string& sec, const std::string& key) const {
        for (const auto& s : sections)
            if (s.first == sec)
                for (const auto& kv : s.second)
                    if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool has_section(const std::string& sec) const {
        for (const auto& s : sections)
            if (s.first == sec) return true;
        return false;
    }
    void set(const std::string& sec, const std::string& key, const std::string& value) {
        for (auto& s : sections)
            if (s.first == sec) {
                for (auto& kv : s.second)
                    if (kv.first == key) { kv.second = value; return; }
                s.second.emplace_back(key, value);
                return;
            }
        sections.push_back({sec, {{key, value}}});
    }
};

inline std::string trim(const std::string& s) {
    size_t a = s.find_first_not_of(" \t\r\n"), b = s.find_last_not_of(" \t\r\n");
    return a == std::string::npos ? std::string() : s.substr(a, b - a + 1);
}

// Returns false and fills `err` on a line the subset does not cover or an unreadable file.
inline bool load(const std::string& path, Doc* doc, std::string* err) {
    std::ifstream f(path);
    if (!f) { *err = "cannot open " + path; return false; }
    std::string line;
    int lineno = 0;
    std::string cur;
    while (std::getline(f, line)) {
        ++lineno;
        // strip comments that are not inside quotes
        bool in_q = false;
        char q = 0;
        for (size_t i = 0; i < line.size(); ++i) {
            char c = line[i];
            if (in_q) { if (c == q) in_q = false; }
            else if (c == '"' || c == '\'') { in_q = true; q = c; }
            else if (c == '#') { line.erase(i); break; }
        }
        if (trim(line).empty()) continue;
        const bool indented = line[0] == ' ' || line[0] == '\t';
        const std::string t = trim(line);
        const size_t colon = t.find(':');
        if (colon == std::string::npos) { *err = path + ":" + std::to_string(lineno) + ": expected 'key: value'"; return false; }
        std::string key = trim(t.substr(0, colon)), val = trim(t.substr(colon + 1));
        if (val.size() >= 2 && (val.front() == '"' || val.front() == '\'') && val.back() == val.front())
            val = val.substr(1, val.size() - 2);
        if (!indented) {
            if (!val.empty()) { *err = path + ":" + std::to_string(lineno) + ": top-level scalars are not part of the schema"; return false; }
            cur = key;
            if (!doc->has_section(cur)) doc->sections.push_back({cur, {}});
        } else {
            if (cur.empty()) { *err = path + ":" + std::to_string(lineno) + ": key outside a section"; return false; }
            doc->set(cur, key, val);
        }
    }
    return true;
}

inline bool save(const std::string& path, const Doc& doc, std::string* err) {
    std::ofstream f(path);
    if (!f) { *err = "cannot write " + path; return false; }
    for (const auto& s : doc.sections) {
        f << s.first << ":\n";
        for (const auto& kv : s.second) f << "  " << kv.first << ": " << kv.second << "\n";
        f << "\n";
    }
    return static_cast<bool>(f);
}

}  // namespace yaml_lite
