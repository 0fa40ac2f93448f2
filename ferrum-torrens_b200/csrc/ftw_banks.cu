// FTW checkpoint index and expert-bank reader (host code only; no kernel in this file).
//
// What it stands in for in the reference engine:
//   src/infrastructure/ftw.rs:63-303     FtwIndex::parse / entry / pieces  (index of `freetoken_weight.json`)
//   src/infrastructure/ftw.rs:346-520    FtwReader::open, WeightsReader::read_range over the shard files
//   src/infrastructure/banks.rs:40-199   bank entry names, read_bank_layer, FtwBanks::slab (one expert's
//                                        three byte fields of `{gate_up,down}_{packed,scale,global}#L{layer:05}`)
// and, on top of them, loading a whole layer straight into an adapter's resident banks (the reference
// stages through pinned host memory and a copy kernel because its experts do not fit the card; here the
// bytes go from the shard files into the slot rows and stay there).
//
// On-disk layout (ftw.rs:1-9): one logical contiguous byte region holding every tensor, cut into shard files;
// every tensor starts at a 4096-aligned region offset; a tensor may span shards.  The index is JSON:
//   {"format": "freetoken_weight", "version": 1, "align": 4096, "total_bytes": N, "shard_limit": N,
//    "tensors": [{"name", "kind", "dtype", "shape", "global_off", "nbytes"}, ..],
//    "shards":  [{"file", "global_off", "nbytes"}, ..], ...}
// Reads are plain positional reads into the caller's buffer (the reference prefers O_DIRECT where the file
// system allows it, to keep a 21 GB cold load out of the page cache; that is a host I/O policy, not part of
// the format, and is left to the host engine).
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "../../include/ftmoe.h"

namespace {

thread_local std::string g_ftw_error;

// ---- a small JSON reader: enough for the index document --------------------------------------
struct JVal {
    enum Type { Null, Bool, Num, Str, Arr, Obj } type = Null;
    bool b = false;
    bool is_uint = false;   // a non-negative integer literal that fits 64 bits
    uint64_t u = 0;
    double d = 0;
    std::string s;
    std::vector<JVal> arr;
    std::vector<std::pair<std::string, JVal>> obj;
    const JVal* get(const char* key) const {
        if (type != Obj) return nullptr;
        for (const auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
};

struct JParser {
    const char* p;
    const char* end;
    std::string err;
    int depth = 0;
    bool fail(const char* what) {
        if (err.empty()) {
            char buf[96];
            snprintf(buf, sizeof buf, "JSON parse failure: %s at byte %zu", what, (size_t)(p - start));
            err = buf;
        }
        return false;
    }
    const char* start;
    void ws() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++;
    }
    bool lit(const char* w) {
        size_t n = strlen(w);
        if ((size_t)(end - p) < n || strncmp(p, w, n) != 0) return fail("unexpected token");
        p += n;
        return true;
    }
    bool str(std::string& out) {
        if (p >= end || *p != '"') return fail("expected a string");
        p++;
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return fail("unterminated escape");
                switch (*p) {
                    case '"': out += '"'; break;
                    case '\\': out += '\\'; break;
                    case '/': out += '/'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'n': out += '\n'; break;
                    case 'r': out += '\r'; break;
                    case 't': out += '\t'; break;
                    case 'u': {
                        if (end - p < 5) return fail("short \\u escape");
                        unsigned cp = 0;
                        for (int i = 1; i <= 4; i++) {
                            char c = p[i];
                            cp <<= 4;
                            if (c >= '0' && c <= '9') cp |= c - '0';
                            else if (c >= 'a' && c <= 'f') cp |= c - 'a' + 10;
                            else if (c >= 'A' && c <= 'F') cp |= c - 'A' + 10;
                            else return fail("bad \\u escape");
                        }
                        p += 4;
                        // names in the index are ASCII; anything else is kept as UTF-8 of the code unit
                        if (cp < 0x80) out += (char)cp;
                        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
                        else { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
                        break;
                    }
                    default: return fail("bad escape");
                }
                p++;
            } else {
                out += *p++;
            }
        }
        if (p >= end) return fail("unterminated string");
        p++;
        return true;
    }
    bool value(JVal& v) {
        if (++depth > 64) return fail("nesting too deep");
        ws();
        if (p >= end) return fail("unexpected end");
        bool ok = true;
        if (*p == '{') {
            v.type = JVal::Obj;
            p++;
            ws();
            if (p < end && *p == '}') { p++; }
            else {
                for (;;) {
                    ws();
                    std::string k;
                    if (!str(k)) { ok = false; break; }
                    ws();
                    if (p >= end || *p != ':') { ok = fail("expected ':'"); break; }
                    p++;
                    JVal child;
                    if (!value(child)) { ok = false; break; }
                    v.obj.emplace_back(std::move(k), std::move(child));
                    ws();
                    if (p < end && *p == ',') { p++; continue; }
                    if (p < end && *p == '}') { p++; break; }
                    ok = fail("expected ',' or '}'");
                    break;
                }
            }
        } else if (*p == '[') {
            v.type = JVal::Arr;
            p++;
            ws();
            if (p < end && *p == ']') { p++; }
            else {
                for (;;) {
                    JVal child;
                    if (!value(child)) { ok = false; break; }
                    v.arr.push_back(std::move(child));
                    ws();
                    if (p < end && *p == ',') { p++; continue; }
                    if (p < end && *p == ']') { p++; break; }
                    ok = fail("expected ',' or ']'");
                    break;
                }
            }
        } else if (*p == '"') {
            v.type = JVal::Str;
            ok = str(v.s);
        } else if (*p == 't') {
            v.type = JVal::Bool; v.b = true; ok = lit("true");
        } else if (*p == 'f') {
            v.type = JVal::Bool; v.b = false; ok = lit("false");
        } else if (*p == 'n') {
            v.type = JVal::Null; ok = lit("null");
        } else {
            const char* q = p;
            bool integer = true;
            if (q < end && *q == '-') { integer = false; q++; }
            if (q >= end || *q < '0' || *q > '9') return fail("unexpected character");
            while (q < end && ((*q >= '0' && *q <= '9') || *q == '.' || *q == 'e' || *q == 'E' || *q == '+' || *q == '-')) {
                if (*q == '.' || *q == 'e' || *q == 'E') integer = false;
                q++;
            }
            std::string num(p, q);
            v.type = JVal::Num;
            v.d = strtod(num.c_str(), nullptr);
            if (integer && num.size() <= 20) {
                errno = 0;
                unsigned long long u = strtoull(num.c_str(), nullptr, 10);
                if (errno == 0) { v.is_uint = true; v.u = u; }
            }
            p = q;
        }
        depth--;
        return ok;
    }
};

// ---- the index ---------------------------------------------------------------------------------
constexpr uint64_t kAlign = 4096;                 // ftw.rs:24
constexpr uint64_t kDefaultShardLimit = 8ull << 30;

struct TensorDesc {
    std::string name, kind, dtype;
    std::vector<uint64_t> shape;
    uint64_t global_off = 0, nbytes = 0;
};
struct ShardDesc {
    std::string file;
    uint64_t global_off = 0, nbytes = 0;
    int fd = -1;
};

// DType::element_size (src/domain/weights.rs:37-45); 0 = unknown dtype name
size_t element_size(const std::string& d) {
    if (d == "bfloat16" || d == "float16") return 2;
    if (d == "float32" || d == "int32") return 4;
    if (d == "float64" || d == "int64") return 8;
    if (d == "float8_e4m3fn" || d == "float8_e4m3fnuz" || d == "int8" || d == "uint8") return 1;
    return 0;
}

int set_err(std::string* dst, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (dst) *dst = buf;
    g_ftw_error = buf;
    return code;
}

}  // namespace

struct ftm_ftw {
    uint64_t shard_limit = kDefaultShardLimit, total_bytes = 0;
    std::vector<TensorDesc> tensors;
    std::vector<ShardDesc> shards;
    bool opened = false;      // shard files are open (ftm_ftw_open); an index parsed from text cannot read
    mutable std::string err;
    const TensorDesc* entry(const std::string& name) const {
        for (const auto& t : tensors)
            if (t.name == name) return &t;
        return nullptr;
    }
    ~ftm_ftw() {
        for (auto& s : shards)
            if (s.fd >= 0) close(s.fd);
    }
};

namespace {

bool get_u64(const JVal* v, uint64_t* out) {
    if (!v || v->type != JVal::Num || !v->is_uint) return false;
    *out = v->u;
    return true;
}

// FtwIndex::parse (ftw.rs:95-252): the same checks in the same order, the same messages
int parse_index(const char* doc, size_t len, ftm_ftw* ix, std::string* err) {
    JParser jp{doc, doc + len, {}, 0, doc};
    JVal v;
    if (!jp.value(v)) return set_err(err, FTM_ERR_READ, "%s", jp.err.c_str());
    jp.ws();
    if (jp.p != jp.end) return set_err(err, FTM_ERR_READ, "JSON parse failure: trailing characters at byte %zu", (size_t)(jp.p - doc));
    if (v.type != JVal::Obj) return set_err(err, FTM_ERR_BAD, "invalid FTW index: missing 'format'");
    const JVal* tag = v.get("format");
    if (!tag || tag->type != JVal::Str) return set_err(err, FTM_ERR_BAD, "invalid FTW index: missing 'format'");
    if (tag->s != "freetoken_weight") return set_err(err, FTM_ERR_BAD, "not an FTW checkpoint: format=\"%s\"", tag->s.c_str());
    uint64_t version = 0, align = 0;
    if (!get_u64(v.get("version"), &version)) return set_err(err, FTM_ERR_BAD, "invalid FTW index: missing 'version'");
    if (version != 1) return set_err(err, FTM_ERR_BAD, "unsupported FTW version %llu", (unsigned long long)version);
    if (!get_u64(v.get("align"), &align)) return set_err(err, FTM_ERR_BAD, "invalid FTW index: missing 'align'");
    if (align != kAlign) return set_err(err, FTM_ERR_BAD, "unexpected alignment %llu; FTW requires %llu", (unsigned long long)align, (unsigned long long)kAlign);
    if (!get_u64(v.get("shard_limit"), &ix->shard_limit)) ix->shard_limit = kDefaultShardLimit;
    if (!get_u64(v.get("total_bytes"), &ix->total_bytes)) return set_err(err, FTM_ERR_BAD, "invalid FTW index: missing 'total_bytes'");
    const JVal* ts = v.get("tensors");
    if (!ts || ts->type != JVal::Arr) return set_err(err, FTM_ERR_BAD, "invalid FTW index: missing 'tensors'");
    for (const JVal& t : ts->arr) {
        TensorDesc d;
        const JVal* name = t.get("name");
        if (!name || name->type != JVal::Str) return set_err(err, FTM_ERR_BAD, "invalid FTW index: tensor missing 'name'");
        d.name = name->s;
        const JVal* kind = t.get("kind");
        if (!kind || kind->type != JVal::Str) return set_err(err, FTM_ERR_BAD, "invalid FTW index: tensor %s missing 'kind'", d.name.c_str());
        d.kind = kind->s;
        const JVal* dtype = t.get("dtype");
        if (!dtype || dtype->type != JVal::Str) return set_err(err, FTM_ERR_BAD, "invalid FTW index: tensor %s missing 'dtype'", d.name.c_str());
        d.dtype = dtype->s;
        if (element_size(d.dtype) == 0)
            return set_err(err, FTM_ERR_BAD, "invalid FTW index: tensor %s: unknown dtype %s", d.name.c_str(), d.dtype.c_str());
        const JVal* shape = t.get("shape");
        if (!shape || shape->type != JVal::Arr) return set_err(err, FTM_ERR_BAD, "invalid FTW index: tensor %s missing 'shape'", d.name.c_str());
        for (const JVal& dim : shape->arr) {
            uint64_t u;
            if (!get_u64(&dim, &u)) return set_err(err, FTM_ERR_BAD, "invalid FTW index: tensor %s has non-integer shape", d.name.c_str());
            d.shape.push_back(u);
        }
        if (!get_u64(t.get("global_off"), &d.global_off)) return set_err(err, FTM_ERR_BAD, "invalid FTW index: tensor %s missing 'global_off'", d.name.c_str());
        if (!get_u64(t.get("nbytes"), &d.nbytes)) return set_err(err, FTM_ERR_BAD, "invalid FTW index: tensor %s missing 'nbytes'", d.name.c_str());
        ix->tensors.push_back(std::move(d));
    }
    const JVal* ss = v.get("shards");
    if (!ss || ss->type != JVal::Arr) return set_err(err, FTM_ERR_BAD, "invalid FTW index: missing 'shards'");
    for (const JVal& s : ss->arr) {
        ShardDesc d;
        const JVal* file = s.get("file");
        if (!file || file->type != JVal::Str) return set_err(err, FTM_ERR_BAD, "invalid FTW index: shard missing 'file'");
        d.file = file->s;
        if (!get_u64(s.get("global_off"), &d.global_off)) return set_err(err, FTM_ERR_BAD, "invalid FTW index: shard %s missing 'global_off'", d.file.c_str());
        if (!get_u64(s.get("nbytes"), &d.nbytes)) return set_err(err, FTM_ERR_BAD, "invalid FTW index: shard %s missing 'nbytes'", d.file.c_str());
        ix->shards.push_back(std::move(d));
    }
    // shards sorted by global_off and contiguous, covering total_bytes
    bool have_prev = false;
    uint64_t prev_end = 0;
    for (const auto& s : ix->shards) {
        if (s.nbytes == 0) return set_err(err, FTM_ERR_BAD, "invalid FTW index: empty shard %s", s.file.c_str());
        if (have_prev && s.global_off != prev_end)
            return set_err(err, FTM_ERR_BAD, "invalid FTW index: shards not contiguous: %s starts at %llu but previous ends at %llu",
                           s.file.c_str(), (unsigned long long)s.global_off, (unsigned long long)prev_end);
        prev_end = s.global_off + s.nbytes;
        have_prev = true;
    }
    if (have_prev) {
        if (prev_end != ix->total_bytes)
            return set_err(err, FTM_ERR_BAD, "invalid FTW index: shards cover %llu bytes but total_bytes=%llu",
                           (unsigned long long)prev_end, (unsigned long long)ix->total_bytes);
    } else if (ix->total_bytes != 0) {
        return set_err(err, FTM_ERR_BAD, "invalid FTW index: no shards but total_bytes > 0");
    }
    for (const auto& t : ix->tensors) {
        if (t.global_off % kAlign)
            return set_err(err, FTM_ERR_BAD, "invalid FTW index: tensor %s starts at unaligned offset %llu", t.name.c_str(),
                           (unsigned long long)t.global_off);
        if (t.nbytes == 0) return set_err(err, FTM_ERR_BAD, "invalid FTW index: tensor %s is empty", t.name.c_str());
        if (t.global_off + t.nbytes > ix->total_bytes)
            return set_err(err, FTM_ERR_BAD, "invalid FTW index: tensor %s range [%llu..%llu) exceeds total_bytes=%llu", t.name.c_str(),
                           (unsigned long long)t.global_off, (unsigned long long)(t.global_off + t.nbytes),
                           (unsigned long long)ix->total_bytes);
        uint64_t n = element_size(t.dtype);
        for (uint64_t dim : t.shape) n *= dim;
        if (n != t.nbytes)
            return set_err(err, FTM_ERR_BAD, "invalid FTW index: tensor %s shape*elsize %llu != nbytes %llu", t.name.c_str(),
                           (unsigned long long)n, (unsigned long long)t.nbytes);
    }
    return FTM_OK;
}

struct Piece {
    int shard;
    uint64_t file_off, dest_off, length;
};

// FtwIndex::pieces (ftw.rs:262-302)
int pieces_of(const ftm_ftw* f, uint64_t global_off, uint64_t nbytes, std::vector<Piece>* out) {
    uint64_t dest = 0, remaining = nbytes, pos = global_off;
    for (size_t i = 0; i < f->shards.size(); i++) {
        const ShardDesc& sh = f->shards[i];
        const uint64_t s0 = sh.global_off, s1 = s0 + sh.nbytes;
        if (pos >= s1 || remaining == 0) continue;
        if (pos < s0) return set_err(&f->err, FTM_ERR_BAD, "invalid FTW index: FTW gap / misordered shards");
        const uint64_t take = remaining < s1 - pos ? remaining : s1 - pos;
        out->push_back(Piece{(int)i, pos - s0, dest, take});
        pos += take;
        dest += take;
        remaining -= take;
    }
    if (remaining > 0) return set_err(&f->err, FTM_ERR_READ, "FTW tensor range exceeds shards");
    return FTM_OK;
}

int read_range(ftm_ftw* f, uint64_t global_off, uint64_t nbytes, uint8_t* dst, std::string* why) {
    if (!f->opened) {
        if (why) *why = "the index was parsed from text: no shard files are open";
        return FTM_ERR_READ;
    }
    std::vector<Piece> ps;
    int rc = pieces_of(f, global_off, nbytes, &ps);
    if (rc != FTM_OK) {
        if (why) *why = f->err;
        return rc;
    }
    for (const Piece& p : ps) {
        uint64_t done = 0;
        while (done < p.length) {
            ssize_t n = pread(f->shards[p.shard].fd, dst + p.dest_off + done, p.length - done, (off_t)(p.file_off + done));
            if (n < 0 && errno == EINTR) continue;
            if (n <= 0) {
                char buf[160];
                if (n == 0) snprintf(buf, sizeof buf, "short read at %llu+%llu", (unsigned long long)p.file_off, (unsigned long long)done);
                else snprintf(buf, sizeof buf, "io failure: %s", strerror(errno));
                if (why) *why = buf;
                return FTM_ERR_READ;
            }
            done += (uint64_t)n;
        }
    }
    return FTM_OK;
}

const char* const kParts[2] = {"gate_up", "down"};
const char* const kFields[3] = {"packed", "scale", "global"};

std::string bank_entry(const char* prefix, int part, int layer, const char* field) {
    char buf[128];
    snprintf(buf, sizeof buf, "%s%s_%s#L%05d", prefix ? prefix : "", kParts[part], field, layer);
    return buf;
}

}  // namespace

extern "C" {

FTM_API const char* ftm_ftw_last_error(const ftm_ftw* f) { return f ? f->err.c_str() : g_ftw_error.c_str(); }

FTM_API int ftm_ftw_parse(const char* json_doc, ftm_ftw** out) {
    if (!json_doc || !out) return set_err(nullptr, FTM_ERR_BAD, "invalid FTW index: null document");
    *out = nullptr;
    std::unique_ptr<ftm_ftw> f(new ftm_ftw);
    int rc = parse_index(json_doc, strlen(json_doc), f.get(), nullptr);
    if (rc != FTM_OK) return rc;
    *out = f.release();
    return FTM_OK;
}

FTM_API int ftm_ftw_open(const char* dir, ftm_ftw** out) {
    if (!dir || !out) return set_err(nullptr, FTM_ERR_BAD, "invalid FTW index: null path");
    *out = nullptr;
    const std::string root(dir);
    const std::string index_path = root + "/freetoken_weight.json";
    FILE* fp = fopen(index_path.c_str(), "rb");
    if (!fp) return set_err(nullptr, FTM_ERR_READ, "io failure: %s: %s", index_path.c_str(), strerror(errno));
    std::string doc;
    char buf[1 << 16];
    size_t n;
    while ((n = fread(buf, 1, sizeof buf, fp)) > 0) doc.append(buf, n);
    fclose(fp);
    std::unique_ptr<ftm_ftw> f(new ftm_ftw);
    int rc = parse_index(doc.data(), doc.size(), f.get(), nullptr);
    if (rc != FTM_OK) return rc;
    if (f->shards.empty()) return set_err(nullptr, FTM_ERR_BAD, "invalid FTW index: index has no shards");
    for (auto& sh : f->shards) {
        const std::string path = root + "/" + sh.file;
        sh.fd = open(path.c_str(), O_RDONLY | O_CLOEXEC);
        if (sh.fd < 0) return set_err(nullptr, FTM_ERR_READ, "io failure: %s: %s", path.c_str(), strerror(errno));
        struct stat st;
        if (fstat(sh.fd, &st) != 0) return set_err(nullptr, FTM_ERR_READ, "io failure: %s: %s", path.c_str(), strerror(errno));
        if ((uint64_t)st.st_size < sh.nbytes)
            return set_err(nullptr, FTM_ERR_BAD, "invalid FTW index: shard %s is %llu bytes but index claims %llu", sh.file.c_str(),
                           (unsigned long long)st.st_size, (unsigned long long)sh.nbytes);
    }
    f->opened = true;
    *out = f.release();
    return FTM_OK;
}

FTM_API void ftm_ftw_close(ftm_ftw* f) { delete f; }

FTM_API int64_t ftm_ftw_tensor_count(const ftm_ftw* f) { return f ? (int64_t)f->tensors.size() : 0; }
FTM_API int64_t ftm_ftw_shard_count(const ftm_ftw* f) { return f ? (int64_t)f->shards.size() : 0; }
FTM_API uint64_t ftm_ftw_total_bytes(const ftm_ftw* f) { return f ? f->total_bytes : 0; }

FTM_API int ftm_ftw_entry(const ftm_ftw* f, const char* name, uint64_t* global_off, uint64_t* nbytes, uint64_t shape[8],
                          int32_t* ndim, int32_t* is_experts_bank) {
    if (!f || !name) return FTM_ERR_BAD;
    const TensorDesc* t = f->entry(name);
    if (!t) return set_err(&f->err, FTM_ERR_MISSING, "moe: no expert bank entry %s", name);
    if (global_off) *global_off = t->global_off;
    if (nbytes) *nbytes = t->nbytes;
    if (ndim) *ndim = (int32_t)t->shape.size();
    if (shape)
        for (size_t i = 0; i < t->shape.size() && i < 8; i++) shape[i] = t->shape[i];
    if (is_experts_bank) *is_experts_bank = t->kind == "experts_bank" ? 1 : 0;
    return FTM_OK;
}

FTM_API int ftm_ftw_pieces(const ftm_ftw* f, uint64_t global_off, uint64_t nbytes, int32_t max_pieces, int32_t* shard_index,
                           uint64_t* file_off, uint64_t* dest_off, uint64_t* length, int32_t* n_pieces) {
    if (!f || !n_pieces) return FTM_ERR_BAD;
    std::vector<Piece> ps;
    int rc = pieces_of(f, global_off, nbytes, &ps);
    if (rc != FTM_OK) return rc;
    *n_pieces = (int32_t)ps.size();
    for (size_t i = 0; i < ps.size() && (int32_t)i < max_pieces; i++) {
        if (shard_index) shard_index[i] = ps[i].shard;
        if (file_off) file_off[i] = ps[i].file_off;
        if (dest_off) dest_off[i] = ps[i].dest_off;
        if (length) length[i] = ps[i].length;
    }
    return FTM_OK;
}

FTM_API int ftm_ftw_read_range(ftm_ftw* f, uint64_t global_off, uint64_t nbytes, void* dst, size_t dst_len) {
    if (!f || (!dst && nbytes)) return FTM_ERR_BAD;
    if (dst_len < nbytes)
        return set_err(&f->err, FTM_ERR_READ, "read_range buffer too small: %zu < %llu", dst_len, (unsigned long long)nbytes);
    std::string why;
    int rc = read_range(f, global_off, nbytes, (uint8_t*)dst, &why);
    if (rc != FTM_OK) return set_err(&f->err, rc, "%s", why.c_str());
    return FTM_OK;
}

// FtwBanks::slab (banks.rs:95-199): one expert's window of the three entries of a part, with the same checks
FTM_API int ftm_ftw_expert_slab(ftm_ftw* f, const char* bank_prefix, int32_t layer, uint32_t expert, int32_t part,
                                uint8_t* packed, uint8_t* scale, uint8_t* global, const size_t cap[3], size_t lens[3],
                                int32_t* rows_out, int32_t* cols_out) {
    if (!f || part < 0 || part > 1 || layer < 0 || !cap || !lens) return FTM_ERR_BAD;
    const std::string pname = bank_entry(bank_prefix, part, layer, "packed");
    const TensorDesc* pt = f->entry(pname);
    if (!pt || pt->kind != "experts_bank") return set_err(&f->err, FTM_ERR_MISSING, "moe: no expert bank entry %s", pname.c_str());
    if (pt->shape.size() != 3) return set_err(&f->err, FTM_ERR_BAD, "moe: %s shape has %zu dimensions", pname.c_str(), pt->shape.size());
    const uint64_t rows = pt->shape[1], cols = pt->shape[2] * 2;
    uint8_t* const dst[3] = {packed, scale, global};
    const uint64_t want[3] = {rows * cols / 2, rows * cols / 16, rows * 2};
    for (int q = 0; q < 3; q++) {
        const std::string name = bank_entry(bank_prefix, part, layer, kFields[q]);
        const TensorDesc* t = f->entry(name);
        if (!t || t->kind != "experts_bank") return set_err(&f->err, FTM_ERR_MISSING, "moe: no expert bank entry %s", name.c_str());
        if (t->shape.empty()) return set_err(&f->err, FTM_ERR_BAD, "moe: %s has no expert axis", name.c_str());
        const uint64_t experts = t->shape[0];
        if (expert >= experts)
            return set_err(&f->err, FTM_ERR_BAD, "moe: expert %u past %llu in %s", expert, (unsigned long long)experts, name.c_str());
        const uint64_t per = t->nbytes / experts;
        if (per * experts != t->nbytes)
            return set_err(&f->err, FTM_ERR_BAD, "moe: %s is %llu bytes for %llu experts", name.c_str(), (unsigned long long)t->nbytes,
                           (unsigned long long)experts);
        lens[q] = (size_t)per;
        if (per != want[q])
            return set_err(&f->err, FTM_ERR_BAD, "moe: %s#L%05d expert %u: %s holds %llu bytes, %llu expected for %llux%llu",
                           kParts[part], layer, expert, kFields[q], (unsigned long long)per, (unsigned long long)want[q],
                           (unsigned long long)rows, (unsigned long long)cols);
        if (cap[q] < per || !dst[q])
            return set_err(&f->err, FTM_ERR_BAD, "moe: %s: the buffer holds %zu bytes, the expert's window is %llu", name.c_str(), cap[q],
                           (unsigned long long)per);
        std::string why;
        int rc = read_range(f, t->global_off + (uint64_t)expert * per, per, dst[q], &why);
        if (rc != FTM_OK) return set_err(&f->err, FTM_ERR_READ, "moe: read %s: %s", name.c_str(), why.c_str());
    }
    if (rows_out) *rows_out = (int32_t)rows;
    if (cols_out) *cols_out = (int32_t)cols;
    return FTM_OK;
}

// Every expert first_expert .. first_expert + n_experts - 1 of `layer` from the checkpoint into slots
// slot0, slot0 + 1, ..: FtwBanks::slab for both parts, then ExpertSlotStore::load.
FTM_API int ftm_load_layer_from_ftw(ftm_handle* h, ftm_ftw* f, const char* bank_prefix, int32_t layer, int32_t first_expert,
                                    int32_t n_experts, int32_t slot0) {
    if (!h || !f) return FTM_ERR_BAD;
    if (n_experts < 0 || first_expert < 0) return set_err(&f->err, FTM_ERR_BAD, "moe: experts %d .. +%d", first_expert, n_experts);
    std::vector<std::vector<uint8_t>> bufs(FTM_NUM_BANKS);
    size_t lens[FTM_NUM_BANKS];
    for (int b = 0; b < FTM_NUM_BANKS; b++) {
        lens[b] = ftm_bank_row_bytes(h, b);
        bufs[b].resize(lens[b]);
    }
    for (int32_t e = 0; e < n_experts; e++) {
        for (int part = 0; part < 2; part++) {
            size_t got[3];
            const size_t cap[3] = {lens[3 * part], lens[3 * part + 1], lens[3 * part + 2]};
            int rc = ftm_ftw_expert_slab(f, bank_prefix, layer, (uint32_t)(first_expert + e), part, bufs[3 * part].data(),
                                         bufs[3 * part + 1].data(), bufs[3 * part + 2].data(), cap, got, nullptr, nullptr);
            if (rc != FTM_OK) return rc;
            for (int q = 0; q < 3; q++)
                if (got[q] != cap[q])
                    return set_err(&f->err, FTM_ERR_BAD, "moe: %s_%s#L%05d holds %zu bytes per expert, the adapter's bank row is %zu",
                                   kParts[part], kFields[q], layer, got[q], cap[q]);
        }
        const uint8_t* fields[FTM_NUM_BANKS];
        for (int b = 0; b < FTM_NUM_BANKS; b++) fields[b] = bufs[b].data();
        int rc = ftm_load_expert(h, layer, first_expert + e, slot0 + e, fields, lens);
        if (rc != FTM_OK) return set_err(&f->err, rc, "%s", ftm_last_error(h));
    }
    return FTM_OK;
}

}  // extern "C"
