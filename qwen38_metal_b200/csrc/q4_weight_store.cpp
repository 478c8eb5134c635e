// Host side of the projection path (include/q4b_weights.h): the safetensors weight store, the Q4 matrix
// descriptor and the projection API of the reference's NativeWeights, written against the public C ABI of the
// CUDA library (q4b200.h) -- shards are uploaded and projections launched only through those entry points.
//
// Follows, in the reference: src/model.rs:51-197 (store, open), :312-323 (shard path check), :336-416 (header),
// :418-459 (range and affine-group checks); src/native.rs:216-385 (NativeWeights), :5383-5515 (Q4AffineMatrix).
#include "../../include/q4b_weights.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <new>
#include <string>
#include <vector>

#include "q4_json.h"

namespace q4 {
int set_error(int status, const char *message);
}

namespace {

constexpr uint64_t kMaxHeaderBytes = 128ull * 1024 * 1024;  // MAX_SAFETENSORS_HEADER_BYTES, src/model.rs:13
constexpr uint64_t kValuesPerWord = 8, kGroup = 64;

int fail(int status, const char *fmt, ...) {
    char buf[768];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    return q4::set_error(status, buf);
}

struct TensorRec {
    std::string dtype;
    std::vector<uint64_t> shape;
    uint32_t shard_index = 0;
    uint64_t byte_offset = 0, byte_len = 0;
};

struct MappedFile {
    std::string path;
    void *base = nullptr;
    uint64_t len = 0;
};

bool checked_mul(uint64_t a, uint64_t b, uint64_t *out) { return !__builtin_mul_overflow(a, b, out); }
bool checked_add(uint64_t a, uint64_t b, uint64_t *out) { return !__builtin_add_overflow(a, b, out); }

std::string shape_text(const std::vector<uint64_t> &shape) {
    std::string s = "[";
    for (size_t i = 0; i < shape.size(); ++i) s += (i ? ", " : "") + std::to_string(shape[i]);
    return s + "]";
}

int read_text_file(const std::string &path, std::string *out) {
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return fail(Q4B_IO_ERROR, "cannot read %s: %s", path.c_str(), strerror(errno));
    char buf[65536];
    size_t n;
    out->clear();
    while ((n = fread(buf, 1, sizeof buf, f)) > 0) out->append(buf, n);
    const bool bad = ferror(f) != 0;
    fclose(f);
    if (bad) return fail(Q4B_IO_ERROR, "cannot read %s: read error", path.c_str());
    return Q4B_OK;
}

int parse_json_file(const std::string &path, const char *kind, q4json::Value *out) {
    std::string text;
    if (int st = read_text_file(path, &text)) return st;
    std::string err;
    if (!q4json::parse(text.data(), text.size(), out, &err))
        return fail(Q4B_JSON_ERROR, "cannot parse %s at %s: %s", kind, path.c_str(), err.c_str());
    return Q4B_OK;
}

// resolve_shard, src/model.rs:312-323: only plain relative components are accepted
int resolve_shard(const std::string &root, const std::string &name, std::string *out) {
    bool safe = !name.empty() && name[0] != '/';
    size_t pos = 0;
    while (safe && pos <= name.size()) {
        const size_t next = name.find('/', pos);
        const std::string part = name.substr(pos, next == std::string::npos ? std::string::npos : next - pos);
        // an empty component ("a//b", trailing '/') is normalised away by the reference's path iterator
        if (part == "." || part == "..") safe = false;
        if (next == std::string::npos) break;
        pos = next + 1;
    }
    if (!safe) return fail(Q4B_UNSAFE_SHARD_PATH, "weight index contains an unsafe shard path \"%s\"", name.c_str());
    *out = root + "/" + name;
    return Q4B_OK;
}

struct HeaderTensor {
    std::string dtype;
    std::vector<uint64_t> shape;
    uint64_t begin = 0, end = 0;
};

struct ShardHeader {
    std::map<std::string, HeaderTensor> tensors;
    uint64_t data_bytes = 0, data_offset = 0;
};

bool as_u64(const q4json::Value &v, uint64_t *out) {
    if (v.type != q4json::Value::Number || !v.is_u64) return false;
    *out = v.u64;
    return true;
}

// read_safetensors_header, src/model.rs:336-416
int read_safetensors_header(const std::string &path, ShardHeader *out) {
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return fail(Q4B_IO_ERROR, "cannot read %s: %s", path.c_str(), strerror(errno));
    struct stat st;
    if (fstat(fileno(f), &st) != 0) {
        const int e = errno;
        fclose(f);
        return fail(Q4B_IO_ERROR, "cannot read %s: %s", path.c_str(), strerror(e));
    }
    const uint64_t file_bytes = (uint64_t)st.st_size;
    if (file_bytes < 8) {
        fclose(f);
        return fail(Q4B_INVALID_HEADER_LENGTH, "invalid safetensors header length 0 for %s (%llu bytes)", path.c_str(),
                    (unsigned long long)file_bytes);
    }
    uint8_t le[8];
    if (fread(le, 1, 8, f) != 8) {
        fclose(f);
        return fail(Q4B_IO_ERROR, "cannot read %s: short read", path.c_str());
    }
    uint64_t header_bytes = 0;
    for (int i = 7; i >= 0; --i) header_bytes = (header_bytes << 8) | le[i];
    if (header_bytes > kMaxHeaderBytes || header_bytes > file_bytes - 8) {
        fclose(f);
        return fail(Q4B_INVALID_HEADER_LENGTH, "invalid safetensors header length %llu for %s (%llu bytes)",
                    (unsigned long long)header_bytes, path.c_str(), (unsigned long long)file_bytes);
    }
    std::string serialized((size_t)header_bytes, '\0');
    const size_t got = header_bytes ? fread(&serialized[0], 1, (size_t)header_bytes, f) : 0;
    fclose(f);
    if (got != header_bytes) return fail(Q4B_IO_ERROR, "cannot read %s: short read", path.c_str());

    q4json::Value doc;
    std::string err;
    if (!q4json::parse(serialized.data(), serialized.size(), &doc, &err) || doc.type != q4json::Value::Object)
        return fail(Q4B_JSON_ERROR, "cannot parse safetensors header at %s: %s", path.c_str(),
                    err.empty() ? "the header is not an object" : err.c_str());
    for (const auto &entry : doc.object) {
        if (entry.first == "__metadata__") continue;
        const q4json::Value &t = entry.second;
        const q4json::Value *dtype = t.find("dtype"), *shape = t.find("shape"), *offsets = t.find("data_offsets");
        bool ok = dtype && shape && offsets && dtype->type == q4json::Value::String && shape->type == q4json::Value::Array &&
                  offsets->type == q4json::Value::Array && offsets->array.size() == 2;
        HeaderTensor h;
        if (ok) {
            h.dtype = dtype->string;
            for (const q4json::Value &d : shape->array) {
                uint64_t v;
                if (!as_u64(d, &v)) ok = false;
                else h.shape.push_back(v);
            }
            ok = ok && as_u64(offsets->array[0], &h.begin) && as_u64(offsets->array[1], &h.end);
        }
        if (!ok)
            return fail(Q4B_JSON_ERROR, "cannot parse safetensors header at %s: tensor \"%s\" needs dtype, shape and two data_offsets",
                        path.c_str(), entry.first.c_str());
        if (h.dtype.empty() || h.shape.empty())
            return fail(Q4B_INVALID_TENSOR_METADATA, "tensor \"%s\" has invalid metadata in %s", entry.first.c_str(), path.c_str());
        out->tensors[entry.first] = std::move(h);
    }
    out->data_bytes = file_bytes - 8 - header_bytes;
    out->data_offset = 8 + header_bytes;
    return Q4B_OK;
}

void fill_info(const TensorRec &rec, q4b_tensor_info *out) {
    memset(out, 0, sizeof *out);
    snprintf(out->dtype, sizeof out->dtype, "%s", rec.dtype.c_str());
    out->rank = (uint32_t)rec.shape.size();
    for (size_t i = 0; i < rec.shape.size() && i < Q4B_MAX_TENSOR_RANK; ++i) out->shape[i] = rec.shape[i];
    out->shard_index = rec.shard_index;
    out->byte_offset = rec.byte_offset;
    out->byte_len = rec.byte_len;
}

std::vector<uint64_t> info_shape(const q4b_tensor_info &t) {
    return std::vector<uint64_t>(t.shape, t.shape + (t.rank < Q4B_MAX_TENSOR_RANK ? t.rank : Q4B_MAX_TENSOR_RANK));
}

// validate_affine_tensor, src/native.rs:5486-5515
int validate_affine_tensor(const char *weight_name, const char *label, const q4b_tensor_info &t, uint64_t rows, uint64_t groups) {
    if (strcmp(t.dtype, "BF16") != 0 || t.rank != 2 || t.shape[0] != rows || t.shape[1] != groups)
        return fail(Q4B_INVALID_AFFINE_TENSOR, "quantized tensor \"%s\" has %s with dtype \"%s\" and shape %s; expected BF16 [%llu, %llu]",
                    weight_name, label, t.dtype, shape_text(info_shape(t)).c_str(), (unsigned long long)rows,
                    (unsigned long long)groups);
    uint64_t expected;
    if (!checked_mul(rows, groups, &expected) || !checked_mul(expected, 2, &expected))
        return fail(Q4B_DIMENSION_OVERFLOW, "dimension overflow in %s", weight_name);
    if (t.byte_len != expected)
        return fail(Q4B_TENSOR_BYTE_LENGTH, "tensor \"%s.%s\" has %llu bytes, expected %llu", weight_name, label,
                    (unsigned long long)t.byte_len, (unsigned long long)expected);
    return Q4B_OK;
}

// Q4AffineMatrix::from_tensors, src/native.rs:5419-5471. `allow_empty` is set for row-sharded views, where a
// rank may own no row of a narrow projection.
int matrix_from_tensors(const char *name, const q4b_tensor_info &weight, const q4b_tensor_info &scales,
                        const q4b_tensor_info &biases, bool allow_empty, q4b_q4_matrix *out) {
    if (strcmp(weight.dtype, "U32") != 0 || weight.rank != 2)
        return fail(Q4B_INVALID_QUANTIZED_WEIGHT, "quantized weight \"%s\" has dtype \"%s\" and shape %s; expected U32 [rows, columns/8]",
                    name, weight.dtype, shape_text(info_shape(weight)).c_str());
    const uint64_t rows = weight.shape[0], packed_columns = weight.shape[1];
    uint64_t k;
    if (!checked_mul(packed_columns, kValuesPerWord, &k)) return fail(Q4B_DIMENSION_OVERFLOW, "dimension overflow in %s", name);
    if ((rows == 0 && !allow_empty) || k == 0 || k % kGroup != 0)
        return fail(Q4B_INVALID_QUANTIZED_WEIGHT, "quantized weight \"%s\" has dtype \"%s\" and shape %s; expected U32 [rows, columns/8]",
                    name, weight.dtype, shape_text(info_shape(weight)).c_str());
    uint64_t expected;
    if (!checked_mul(rows, packed_columns, &expected) || !checked_mul(expected, 4, &expected))
        return fail(Q4B_DIMENSION_OVERFLOW, "dimension overflow in %s", name);
    if (weight.byte_len != expected)
        return fail(Q4B_TENSOR_BYTE_LENGTH, "tensor \"%s\" has %llu bytes, expected %llu", name, (unsigned long long)weight.byte_len,
                    (unsigned long long)expected);
    const uint64_t groups = k / kGroup;
    if (int st = validate_affine_tensor(name, "scales", scales, rows, groups)) return st;
    if (int st = validate_affine_tensor(name, "biases", biases, rows, groups)) return st;
    const size_t len = strlen(name);
    if (len < 7 || strcmp(name + len - 7, ".weight") != 0)
        return fail(Q4B_NOT_QUANTIZED_WEIGHT, "tensor \"%s\" is not a quantized .weight tensor", name);
    memset(out, 0, sizeof *out);
    out->weight = weight;
    out->scales = scales;
    out->biases = biases;
    out->input_elements = k;
    out->output_rows = rows;
    out->row_begin = 0;
    out->total_rows = rows;
    return Q4B_OK;
}

typedef std::map<std::string, TensorRec> TensorMap;

int matrix_from_map(const TensorMap &tensors, const char *name, bool allow_empty, q4b_q4_matrix *out) {
    const auto w = tensors.find(name);
    if (w == tensors.end()) return fail(Q4B_MISSING_TENSOR, "tensor \"%s\" is absent", name);
    const std::string full(name);
    if (full.size() < 7 || full.compare(full.size() - 7, 7, ".weight") != 0)
        return fail(Q4B_NOT_QUANTIZED_WEIGHT, "tensor \"%s\" is not a quantized .weight tensor", name);
    const std::string base = full.substr(0, full.size() - 7);
    const auto s = tensors.find(base + ".scales");
    if (s == tensors.end()) return fail(Q4B_MISSING_TENSOR, "tensor \"%s.scales\" is absent", base.c_str());
    const auto b = tensors.find(base + ".biases");
    if (b == tensors.end()) return fail(Q4B_MISSING_TENSOR, "tensor \"%s.biases\" is absent", base.c_str());
    for (const auto *rec : {&w->second, &s->second, &b->second})
        if (rec->shape.size() > Q4B_MAX_TENSOR_RANK)
            return fail(Q4B_UNSUPPORTED, "tensor rank %zu exceeds %d", rec->shape.size(), Q4B_MAX_TENSOR_RANK);
    q4b_tensor_info wi, si, bi;
    fill_info(w->second, &wi);
    fill_info(s->second, &si);
    fill_info(b->second, &bi);
    return matrix_from_tensors(name, wi, si, bi, allow_empty, out);
}

}  // namespace

struct q4b_store {
    std::vector<MappedFile> shards;
    TensorMap tensors;
    std::vector<const std::string *> names;  // sorted (map order)
    uint64_t indexed_tensor_bytes = 0;
    uint64_t quantized_groups = 0;
    ~q4b_store() {
        for (MappedFile &m : shards)
            if (m.base) munmap(m.base, (size_t)m.len);
    }
};

struct q4b_weights {
    q4b_runtime *rt = nullptr;
    q4b_store *store = nullptr;
    std::vector<uint32_t> shard_ids;  // device shard of store shard i
    TensorMap device_tensors;         // what sits in HBM: the store's records, or this rank's row slices
    uint32_t rank = 0, world = 1;
    uint64_t device_bytes = 0;
};

// ------------------------------------------------------------------------------------------------
// store
// ------------------------------------------------------------------------------------------------

extern "C" int q4b_store_open(const char *directory, q4b_store **out) {
    if (!directory || !out) return fail(Q4B_INVALID_ARGUMENT, "directory or output pointer is null");
    const std::string root(directory);

    // the quantisation block of config.json (inspect_mlx_safetensors_dir, src/model.rs:229-240)
    q4json::Value config;
    if (int st = parse_json_file(root + "/config.json", "config.json", &config)) return st;
    const q4json::Value *quant = config.find("quantization_config");
    if (!quant || quant->type != q4json::Value::Object) quant = config.find("quantization");
    if (!quant || quant->type != q4json::Value::Object)
        return fail(Q4B_MISSING_QUANTIZATION, "model config does not declare MLX quantization");
    {
        const q4json::Value *bits = quant->find("bits"), *group = quant->find("group_size"), *mode = quant->find("mode");
        uint64_t b = 0, g = 0;
        if (!bits || !group || !mode || !as_u64(*bits, &b) || !as_u64(*group, &g) || mode->type != q4json::Value::String || b > 255 ||
            g > 0xffffffffull)
            return fail(Q4B_JSON_ERROR, "cannot parse config.json at %s/config.json: quantization needs bits, group_size and mode",
                        root.c_str());
        if (b != 4 || g == 0 || mode->string != "affine")
            return fail(Q4B_UNSUPPORTED_QUANTIZATION, "unsupported quantization bits=%llu, group_size=%llu, mode=\"%s\"; expected 4-bit affine",
                        (unsigned long long)b, (unsigned long long)g, mode->string.c_str());
    }

    q4json::Value index;
    const std::string index_path = root + "/model.safetensors.index.json";
    if (int st = parse_json_file(index_path, "model.safetensors.index.json", &index)) return st;
    std::map<std::string, std::string> weight_map;
    if (index.type != q4json::Value::Object)
        return fail(Q4B_JSON_ERROR, "cannot parse model.safetensors.index.json at %s: the index is not an object", index_path.c_str());
    if (const q4json::Value *wm = index.find("weight_map")) {
        if (wm->type != q4json::Value::Object)
            return fail(Q4B_JSON_ERROR, "cannot parse model.safetensors.index.json at %s: weight_map is not an object", index_path.c_str());
        for (const auto &entry : wm->object) {
            if (entry.second.type != q4json::Value::String)
                return fail(Q4B_JSON_ERROR, "cannot parse model.safetensors.index.json at %s: shard of \"%s\" is not a string",
                            index_path.c_str(), entry.first.c_str());
            weight_map[entry.first] = entry.second.string;
        }
    }
    std::map<std::string, std::vector<std::string>> by_shard;
    for (const auto &entry : weight_map) by_shard[entry.second].push_back(entry.first);

    q4b_store *store = new (std::nothrow) q4b_store();
    if (!store) return fail(Q4B_CUDA_ERROR, "out of host memory");
    int status = Q4B_OK;
    for (const auto &group : by_shard) {
        std::string path;
        if ((status = resolve_shard(root, group.first, &path))) break;
        ShardHeader header;
        if ((status = read_safetensors_header(path, &header))) break;
        const uint32_t shard_index = (uint32_t)store->shards.size();
        for (const std::string &name : group.second) {
            const auto it = header.tensors.find(name);
            if (it == header.tensors.end()) {
                status = fail(Q4B_MISSING_INDEXED_TENSOR, "weight index tensor \"%s\" is absent from %s", name.c_str(), path.c_str());
                break;
            }
            const HeaderTensor &t = it->second;
            // validate_tensor_range, src/model.rs:418-431
            if (t.begin > t.end || t.end > header.data_bytes) {
                status = fail(Q4B_INVALID_TENSOR_OFFSETS, "tensor \"%s\" has offsets outside the data section of %s", name.c_str(),
                              path.c_str());
                break;
            }
            TensorRec rec;
            rec.dtype = t.dtype;
            rec.shape = t.shape;
            rec.shard_index = shard_index;
            if (!checked_add(header.data_offset, t.begin, &rec.byte_offset)) {
                status = fail(Q4B_DIMENSION_OVERFLOW, "model tensor size overflows u64");
                break;
            }
            rec.byte_len = t.end - t.begin;
            if (!checked_add(store->indexed_tensor_bytes, rec.byte_len, &store->indexed_tensor_bytes)) {
                status = fail(Q4B_DIMENSION_OVERFLOW, "model tensor size overflows u64");
                break;
            }
            store->tensors[name] = std::move(rec);
        }
        if (status) break;
        const int fd = open(path.c_str(), O_RDONLY);
        if (fd < 0) {
            status = fail(Q4B_IO_ERROR, "cannot read %s: %s", path.c_str(), strerror(errno));
            break;
        }
        struct stat st;
        void *base = MAP_FAILED;
        if (fstat(fd, &st) == 0) base = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
        const int map_errno = errno;
        close(fd);
        if (base == MAP_FAILED) {
            status = fail(Q4B_IO_ERROR, "cannot read %s: %s", path.c_str(), strerror(map_errno));
            break;
        }
        MappedFile m;
        m.path = path;
        m.base = base;
        m.len = (uint64_t)st.st_size;
        store->shards.push_back(m);
    }
    // validate_affine_groups, src/model.rs:433-459
    if (!status) {
        for (const auto &entry : weight_map) {
            const std::string &name = entry.first;
            if (name.size() < 7 || name.compare(name.size() - 7, 7, ".weight") != 0) continue;
            const std::string base = name.substr(0, name.size() - 7);
            const bool has_scales = weight_map.count(base + ".scales") != 0, has_biases = weight_map.count(base + ".biases") != 0;
            if (has_scales != has_biases) {
                status = fail(Q4B_INCOMPLETE_AFFINE_GROUP, "quantized tensor \"%s\" is missing its affine %s companion", name.c_str(),
                              has_scales ? "biases" : "scales");
                break;
            }
            if (has_scales) store->quantized_groups++;
        }
    }
    if (status) {
        delete store;
        return status;
    }
    for (const auto &entry : store->tensors) store->names.push_back(&entry.first);
    *out = store;
    return Q4B_OK;
}

extern "C" void q4b_store_close(q4b_store *store) { delete store; }

#define Q4B_STORE_COUNTER(fn, expr)                                                           \
    extern "C" int fn(const q4b_store *store, uint64_t *out) {                                \
        if (!store || !out) return fail(Q4B_INVALID_ARGUMENT, "store or output pointer is null"); \
        *out = (expr);                                                                        \
        return Q4B_OK;                                                                        \
    }
Q4B_STORE_COUNTER(q4b_store_tensor_count, store->tensors.size())
Q4B_STORE_COUNTER(q4b_store_shard_count, store->shards.size())
Q4B_STORE_COUNTER(q4b_store_indexed_tensor_bytes, store->indexed_tensor_bytes)
Q4B_STORE_COUNTER(q4b_store_quantized_groups, store->quantized_groups)

extern "C" int q4b_store_mapped_bytes(const q4b_store *store, uint64_t *out) {
    if (!store || !out) return fail(Q4B_INVALID_ARGUMENT, "store or output pointer is null");
    uint64_t total = 0;
    for (const MappedFile &m : store->shards) total += m.len;
    *out = total;
    return Q4B_OK;
}

extern "C" int q4b_store_tensor(const q4b_store *store, const char *name, q4b_tensor_info *out) {
    if (!store || !name || !out) return fail(Q4B_INVALID_ARGUMENT, "store, name or output pointer is null");
    const auto it = store->tensors.find(name);
    if (it == store->tensors.end()) return fail(Q4B_MISSING_TENSOR, "runtime tensor \"%s\" is absent", name);
    if (it->second.shape.size() > Q4B_MAX_TENSOR_RANK)
        return fail(Q4B_UNSUPPORTED, "tensor rank %zu exceeds %d", it->second.shape.size(), Q4B_MAX_TENSOR_RANK);
    fill_info(it->second, out);
    return Q4B_OK;
}

extern "C" int q4b_store_tensor_name(const q4b_store *store, uint64_t index, const char **name) {
    if (!store || !name) return fail(Q4B_INVALID_ARGUMENT, "store or output pointer is null");
    if (index >= store->names.size()) return fail(Q4B_MISSING_TENSOR, "tensor index %llu is past the end", (unsigned long long)index);
    *name = store->names[index]->c_str();
    return Q4B_OK;
}

// MlxWeightStore::tensor_bytes, src/model.rs:79-85
static int tensor_bytes(const q4b_store *store, const TensorRec &rec, const char *name, const uint8_t **data) {
    if (rec.shard_index >= store->shards.size()) return fail(Q4B_INVALID_RUNTIME_TENSOR, "runtime tensor \"%s\" has an invalid byte range", name);
    const MappedFile &m = store->shards[rec.shard_index];
    uint64_t end;
    if (!checked_add(rec.byte_offset, rec.byte_len, &end) || end > m.len)
        return fail(Q4B_INVALID_RUNTIME_TENSOR, "runtime tensor \"%s\" has an invalid byte range", name);
    *data = (const uint8_t *)m.base + rec.byte_offset;
    return Q4B_OK;
}

extern "C" int q4b_store_tensor_data(const q4b_store *store, const char *name, const void **data, uint64_t *len) {
    if (!store || !name || !data || !len) return fail(Q4B_INVALID_ARGUMENT, "store, name or output pointer is null");
    const auto it = store->tensors.find(name);
    if (it == store->tensors.end()) return fail(Q4B_MISSING_TENSOR, "runtime tensor \"%s\" is absent", name);
    const uint8_t *p = nullptr;
    if (int st = tensor_bytes(store, it->second, name, &p)) return st;
    *data = p;
    *len = it->second.byte_len;
    return Q4B_OK;
}

extern "C" int q4b_store_shard_data(const q4b_store *store, uint64_t shard_index, const void **data, uint64_t *len) {
    if (!store || !data || !len) return fail(Q4B_INVALID_ARGUMENT, "store or output pointer is null");
    if (shard_index >= store->shards.size()) return fail(Q4B_MISSING_SHARD, "mapped safetensors shard %llu is absent", (unsigned long long)shard_index);
    *data = store->shards[shard_index].base;
    *len = store->shards[shard_index].len;
    return Q4B_OK;
}

extern "C" int q4b_store_tensor_values_f32(const q4b_store *store, const char *name, float *out, uint64_t capacity, uint64_t *count) {
    if (!store || !name || !count) return fail(Q4B_INVALID_ARGUMENT, "store, name or count pointer is null");
    const auto it = store->tensors.find(name);
    if (it == store->tensors.end()) return fail(Q4B_MISSING_TENSOR, "runtime tensor \"%s\" is absent", name);
    const uint8_t *p = nullptr;
    if (int st = tensor_bytes(store, it->second, name, &p)) return st;
    const TensorRec &rec = it->second;
    uint64_t width;
    if (rec.dtype == "BF16") width = 2;
    else if (rec.dtype == "F32") width = 4;
    else
        return fail(Q4B_UNSUPPORTED_DTYPE, "runtime tensor \"%s\" uses unsupported dtype \"%s\"; expected BF16 or F32", name, rec.dtype.c_str());
    const uint64_t n = rec.byte_len / width;  // chunks_exact: a ragged tail is dropped
    *count = n;
    if (!out) return Q4B_OK;  // size query
    if (capacity < n) return fail(Q4B_WRONG_LENGTH, "output has %llu elements, expected %llu", (unsigned long long)capacity, (unsigned long long)n);
    for (uint64_t i = 0; i < n; ++i) {
        uint32_t bits;
        if (width == 2) bits = ((uint32_t)p[2 * i] | ((uint32_t)p[2 * i + 1] << 8)) << 16;
        else bits = (uint32_t)p[4 * i] | ((uint32_t)p[4 * i + 1] << 8) | ((uint32_t)p[4 * i + 2] << 16) | ((uint32_t)p[4 * i + 3] << 24);
        memcpy(out + i, &bits, 4);
    }
    return Q4B_OK;
}

extern "C" int q4b_store_q4_matrix(const q4b_store *store, const char *weight_name, q4b_q4_matrix *out) {
    if (!store || !weight_name || !out) return fail(Q4B_INVALID_ARGUMENT, "store, name or output pointer is null");
    return matrix_from_map(store->tensors, weight_name, false, out);
}

extern "C" int q4b_q4_matrix_from_tensors(const char *weight_name, const q4b_tensor_info *weight, const q4b_tensor_info *scales,
                                          const q4b_tensor_info *biases, q4b_q4_matrix *out) {
    if (!weight_name || !weight || !scales || !biases || !out) return fail(Q4B_INVALID_ARGUMENT, "a pointer argument is null");
    return matrix_from_tensors(weight_name, *weight, *scales, *biases, false, out);
}

// ------------------------------------------------------------------------------------------------
// weights in HBM
// ------------------------------------------------------------------------------------------------

namespace {

void release_weights(q4b_weights *w) {
    if (!w) return;
    for (uint32_t id : w->shard_ids) q4b_shard_free(w->rt, id);
    delete w->store;
    delete w;
}

struct Piece {
    uint64_t src_offset, bytes, dst_offset;
};

}  // namespace

extern "C" int q4b_weights_open_sharded(q4b_runtime *rt, const char *directory, uint32_t rank, uint32_t world, q4b_weights **out) {
    if (!rt || !out) return fail(Q4B_INVALID_ARGUMENT, "runtime or output pointer is null");
    if (world == 0 || rank >= world) return fail(Q4B_INVALID_ARGUMENT, "rank %u is not below world size %u", rank, world);
    q4b_store *store = nullptr;
    if (int st = q4b_store_open(directory, &store)) return st;
    q4b_weights *w = new (std::nothrow) q4b_weights();
    if (!w) {
        delete store;
        return fail(Q4B_CUDA_ERROR, "out of host memory");
    }
    w->rt = rt;
    w->store = store;
    w->rank = rank;
    w->world = world;

    if (world == 1) {
        // map_weight_store, src/metal_runtime.rs:955-982: every shard whole, file offsets kept
        for (const MappedFile &m : store->shards) {
            uint32_t id = 0;
            if (int st = q4b_shard_upload(rt, m.base, m.len, &id)) {
                release_weights(w);
                return st;
            }
            w->shard_ids.push_back(id);
            w->device_bytes += m.len;
        }
        w->device_tensors = store->tensors;
        *out = w;
        return Q4B_OK;
    }

    // Row-sharded: which tensors belong to a quantised projection (sliced by rows) and which are kept whole
    std::map<std::string, uint64_t> sliced_rows;  // tensor name -> total rows, for members of valid Q4 groups
    for (const auto &entry : store->tensors) {
        const std::string &name = entry.first;
        if (name.size() < 7 || name.compare(name.size() - 7, 7, ".weight") != 0) continue;
        const std::string base = name.substr(0, name.size() - 7);
        if (!store->tensors.count(base + ".scales") || !store->tensors.count(base + ".biases")) continue;
        q4b_q4_matrix m;
        if (matrix_from_map(store->tensors, name.c_str(), false, &m) != Q4B_OK) continue;  // not a Q4 projection: kept whole
        sliced_rows[name] = sliced_rows[base + ".scales"] = sliced_rows[base + ".biases"] = m.output_rows;
    }
    std::vector<std::vector<const std::string *>> per_shard(store->shards.size());
    for (const auto &entry : store->tensors) per_shard[entry.second.shard_index].push_back(&entry.first);
    for (size_t si = 0; si < store->shards.size(); ++si) {
        std::vector<const std::string *> &names = per_shard[si];
        std::sort(names.begin(), names.end(), [&](const std::string *a, const std::string *b) {
            return store->tensors[*a].byte_offset < store->tensors[*b].byte_offset;
        });
        std::vector<Piece> pieces;
        uint64_t pos = 0;
        for (const std::string *name : names) {
            const TensorRec &src = store->tensors[*name];
            TensorRec dst = src;
            uint64_t begin = 0, bytes = src.byte_len;
            const auto sl = sliced_rows.find(*name);
            if (sl != sliced_rows.end()) {
                const uint64_t rows = sl->second, row_bytes = src.byte_len / rows;
                const uint64_t r0 = rows * rank / world, r1 = rows * (rank + 1) / world;
                begin = r0 * row_bytes;
                bytes = (r1 - r0) * row_bytes;
                dst.shape[0] = r1 - r0;
            }
            // same address modulo 16 as in the file (device allocations are at least 256-byte aligned)
            const uint64_t want = (src.byte_offset + begin) & 15u;
            pos = ((pos + 15u) & ~15ull) + want;
            dst.shard_index = (uint32_t)si;
            dst.byte_offset = pos;
            dst.byte_len = bytes;
            if (bytes) pieces.push_back(Piece{src.byte_offset + begin, bytes, pos});
            pos += bytes;
            w->device_tensors[*name] = std::move(dst);
        }
        uint32_t id = 0;
        int st = q4b_shard_alloc(rt, pos ? pos : 16, &id);
        if (!st) {
            w->shard_ids.push_back(id);
            for (const Piece &p : pieces) {
                st = q4b_shard_write(rt, id, p.dst_offset, (const uint8_t *)store->shards[si].base + p.src_offset, p.bytes);
                if (st) break;
                w->device_bytes += p.bytes;
            }
        }
        if (st) {
            release_weights(w);
            return st;
        }
    }
    // global row range of every sliced tensor is recomputed on demand in q4b_weights_q4_matrix
    *out = w;
    return Q4B_OK;
}

extern "C" int q4b_weights_open(q4b_runtime *rt, const char *directory, q4b_weights **out) {
    return q4b_weights_open_sharded(rt, directory, 0, 1, out);
}

extern "C" void q4b_weights_close(q4b_weights *weights) { release_weights(weights); }

extern "C" int q4b_weights_store(q4b_weights *weights, q4b_store **out) {
    if (!weights || !out) return fail(Q4B_INVALID_ARGUMENT, "weights or output pointer is null");
    *out = weights->store;
    return Q4B_OK;
}

extern "C" int q4b_weights_shard_count(const q4b_weights *weights, uint64_t *out) {
    if (!weights || !out) return fail(Q4B_INVALID_ARGUMENT, "weights or output pointer is null");
    *out = weights->shard_ids.size();
    return Q4B_OK;
}

extern "C" int q4b_weights_device_bytes(const q4b_weights *weights, uint64_t *out) {
    if (!weights || !out) return fail(Q4B_INVALID_ARGUMENT, "weights or output pointer is null");
    *out = weights->device_bytes;
    return Q4B_OK;
}

extern "C" int q4b_weights_q4_matrix(const q4b_weights *weights, const char *weight_name, q4b_q4_matrix *out) {
    if (!weights || !weight_name || !out) return fail(Q4B_INVALID_ARGUMENT, "weights, name or output pointer is null");
    if (int st = matrix_from_map(weights->device_tensors, weight_name, weights->world > 1, out)) return st;
    if (weights->world > 1) {
        const auto it = weights->store->tensors.find(weight_name);
        const uint64_t total = it->second.shape[0];
        out->total_rows = total;
        out->row_begin = total * weights->rank / weights->world;
    }
    return Q4B_OK;
}

// NativeWeights::mapped_q4_jobs, src/native.rs:325-382
extern "C" int q4b_weights_jobs(const q4b_weights *weights, const q4b_q4_matrix *matrices, uint32_t n, uint64_t input_elements,
                                q4b_job *jobs) {
    if (!weights || !jobs || (!matrices && n)) return fail(Q4B_INVALID_ARGUMENT, "weights, matrices or jobs pointer is null");
    if (n == 0) return fail(Q4B_INVALID_CONFIG, "a Q4 projection batch requires at least one matrix");
    std::vector<q4b_job> built(n);
    for (uint32_t i = 0; i < n; ++i) {
        const q4b_q4_matrix &m = matrices[i];
        if (input_elements != m.input_elements)
            return fail(Q4B_INPUT_DIMENSION, "input has %llu elements, the projection expects %llu", (unsigned long long)input_elements,
                        (unsigned long long)m.input_elements);
        if (m.output_rows == 0) return fail(Q4B_EMPTY_DIMENSION, "this rank owns no row of projection %u", i);
        const q4b_tensor_info *parts[3] = {&m.weight, &m.scales, &m.biases};
        uint32_t ids[3];
        int aligned = 1;
        const uint64_t need[3] = {4, 2, 2};
        for (int p = 0; p < 3; ++p) {
            if (parts[p]->shard_index >= weights->shard_ids.size())
                return fail(Q4B_MISSING_SHARD, "mapped safetensors shard %u is absent", parts[p]->shard_index);
            ids[p] = weights->shard_ids[parts[p]->shard_index];
            int ok = 0;
            if (int st = q4b_offset_is_aligned(weights->rt, ids[p], parts[p]->byte_offset, need[p], &ok)) return st;
            aligned = aligned && ok;
        }
        q4b_job &j = built[i];
        j.weight_shard = ids[0];
        j.scale_shard = ids[1];
        j.bias_shard = ids[2];
        j.aligned = aligned;
        j.weight_offset = m.weight.byte_offset;
        j.scale_offset = m.scales.byte_offset;
        j.bias_offset = m.biases.byte_offset;
        j.output_rows = m.output_rows;
    }
    memcpy(jobs, built.data(), sizeof(q4b_job) * n);
    return Q4B_OK;
}

static int check_batch(const char *what, const float *x, uint64_t x_len, uint64_t batch_size) {
    if (batch_size == 0 || x_len == 0 || x_len % batch_size != 0) return fail(Q4B_INVALID_CONFIG, "%s needs non-empty, evenly sized rows", what);
    if (!x) return fail(Q4B_INVALID_ARGUMENT, "input pointer is null");
    return Q4B_OK;
}

extern "C" int q4b_weights_matvec_batch(const q4b_weights *weights, const q4b_q4_matrix *matrices, uint32_t n, const float *x,
                                        uint64_t x_len, float *const *outputs) {
    if (!weights) return fail(Q4B_INVALID_ARGUMENT, "weights pointer is null");
    std::vector<q4b_job> jobs(n ? n : 1);
    if (int st = q4b_weights_jobs(weights, matrices, n, x_len, jobs.data())) return st;
    return q4b_matvec_batch(weights->rt, x, Q4B_F32, x_len, jobs.data(), n, outputs);
}

extern "C" int q4b_weights_matmul_batch(const q4b_weights *weights, const q4b_q4_matrix *matrices, uint32_t n, const float *x,
                                        uint64_t x_len, uint64_t batch_size, float *const *outputs) {
    if (!weights) return fail(Q4B_INVALID_ARGUMENT, "weights pointer is null");
    if (int st = check_batch("a Q4 prefill batch", x, x_len, batch_size)) return st;
    std::vector<q4b_job> jobs(n ? n : 1);
    const uint64_t k = x_len / batch_size;
    if (int st = q4b_weights_jobs(weights, matrices, n, k, jobs.data())) return st;
    return q4b_matmul_batch(weights->rt, x, Q4B_F32, batch_size, k, jobs.data(), n, outputs);
}

extern "C" int q4b_weights_argmax_batch(const q4b_weights *weights, const q4b_q4_matrix *matrix, const float *x, uint64_t x_len,
                                        uint64_t batch_size, uint32_t *tokens) {
    if (!weights || !matrix) return fail(Q4B_INVALID_ARGUMENT, "weights or matrix pointer is null");
    if (int st = check_batch("a Q4 argmax batch", x, x_len, batch_size)) return st;
    q4b_job job;
    const uint64_t k = x_len / batch_size;
    if (int st = q4b_weights_jobs(weights, matrix, 1, k, &job)) return st;
    return q4b_argmax_batch(weights->rt, x, Q4B_F32, batch_size, k, &job, tokens);
}

extern "C" int q4b_weights_mlp_batch(const q4b_weights *weights, const q4b_q4_matrix *gate, const q4b_q4_matrix *up,
                                     const q4b_q4_matrix *down, const float *x, uint64_t x_len, uint64_t batch_size, float *out) {
    if (!weights || !gate || !up || !down) return fail(Q4B_INVALID_ARGUMENT, "weights or matrix pointer is null");
    if (int st = check_batch("an MLP prefill batch", x, x_len, batch_size)) return st;
    const uint64_t k = x_len / batch_size;
    const q4b_q4_matrix pair[2] = {*gate, *up};
    q4b_job gu[2], dj;
    if (int st = q4b_weights_jobs(weights, pair, 2, k, gu)) return st;
    if (int st = q4b_weights_jobs(weights, down, 1, gate->output_rows, &dj)) return st;
    return q4b_mlp_batch(weights->rt, x, Q4B_F32, batch_size, k, &gu[0], &gu[1], &dj, out);
}

extern "C" int q4b_weights_dequantized_row(const q4b_weights *weights, const q4b_q4_matrix *matrix, uint64_t row, float *out) {
    if (!weights || !matrix || !out) return fail(Q4B_INVALID_ARGUMENT, "weights, matrix or output pointer is null");
    if (row >= matrix->output_rows) return fail(Q4B_TOKEN_OUT_OF_RANGE, "token %llu is outside the matrix", (unsigned long long)row);
    q4b_job job;
    if (int st = q4b_weights_jobs(weights, matrix, 1, matrix->input_elements, &job)) return st;
    return q4b_dequantize_row(weights->rt, &job, matrix->input_elements, row, out);
}
