// The QIPACK v6 container on the host: reading a pack's header, directory and metadata, verifying it the way the
// reference's packer does, handing out a record as the run-time view the kernels take, and writing a pack from
// tensors that are already quantised. Layout and rules follow qwen_image_cuda/src/int4_pack.cplus:36-95
// (PackedHeader, PackedRecord, 256 bytes each, little-endian), :151-159 (FNV-1a), :476-518 (plan_record: every
// region 256-byte aligned, weights then scales then zeros), :628-666 (payload and metadata checksums, metadata in
// the directory padding), :733-850 (verify) and the metadata reader qwen_image/src/pack_info.cplus:22-145.
// Quantising weights is not done here: the engine's packs are written offline by the reference's packer.
#pragma once

#include <errno.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <string>
#include <vector>

#include "../../include/qipack_b200.h"

namespace qi {
namespace pack {

constexpr uint64_t HEADER_BYTES = 256, RECORD_BYTES = 256, TENSOR_ALIGNMENT = 256;
constexpr uint64_t FNV_OFFSET = 14695981039346656037ull, FNV_PRIME = 1099511628211ull;
constexpr uint32_t SCHEME_BF16 = 0, SCHEME_FP16 = 1, TYPE_NONE = 0, TYPE_F16 = 1, METADATA_VERSION = 1;
constexpr size_t IO_CHUNK = 1u << 24;

#pragma pack(push, 1)
struct Header {  // int4_pack.cplus:56-74
    uint8_t magic[8];
    uint32_t version, header_bytes, tensor_count, scope;
    uint64_t directory_offset, data_offset, file_bytes, payload_checksum;
    uint8_t model_snapshot[40], diffusers_commit[40], policy[32];
    uint64_t metadata_offset;
    uint32_t metadata_bytes, metadata_version;
    uint64_t metadata_checksum;
    uint8_t reserved[64];
};
struct Record {  // int4_pack.cplus:76-95
    uint8_t name[128];
    uint32_t scheme, rank;
    uint64_t dimensions[4];
    uint32_t group_axis, group_size, scale_type, zero_type;
    uint64_t weights_offset, weights_length, scales_offset, scales_length, zeros_offset, zeros_length;
    uint64_t elements, tensor_checksum;
    uint8_t reserved[8];
};
#pragma pack(pop)
static_assert(sizeof(Header) == HEADER_BYTES && sizeof(Record) == RECORD_BYTES, "the container's fixed layouts");

const uint8_t MAGIC[8] = {'Q', 'I', 'P', 'A', 'C', 'K', '1', 0};

inline uint64_t align_up(uint64_t value, uint64_t alignment) { return (value + alignment - 1) / alignment * alignment; }

inline uint64_t hash_update(uint64_t hash, const uint8_t *bytes, size_t count) {  // int4_pack.cplus:151-159
    for (size_t i = 0; i < count; ++i) hash = (hash ^ bytes[i]) * FNV_PRIME;
    return hash;
}

inline bool read_exact(FILE *file, void *out, size_t bytes, uint64_t offset) {
    if (fseeko(file, static_cast<off_t>(offset), SEEK_SET) != 0) return false;
    return fread(out, 1, bytes, file) == bytes;
}

inline bool write_exact(FILE *file, const void *in, size_t bytes, uint64_t offset) {
    if (fseeko(file, static_cast<off_t>(offset), SEEK_SET) != 0) return false;
    return fwrite(in, 1, bytes, file) == bytes;
}

inline std::string fixed_string(const uint8_t *bytes, size_t capacity) {
    size_t length = 0;
    while (length < capacity && bytes[length] != 0) ++length;
    return std::string(reinterpret_cast<const char *>(bytes), length);
}

inline bool fixed_text(uint8_t *out, size_t capacity, const char *text) {  // zero-padded, int4_pack.cplus:191-206
    const size_t length = strlen(text);
    if (length > capacity) return false;
    memset(out, 0, capacity);
    memcpy(out, text, length);
    return true;
}

// which quantised scheme a policy string announces (int4_pack.cplus:753-764), 0 for none
inline uint32_t policy_scheme(const std::string &policy) {
    for (const char *group : {"32", "64", "128"}) {
        if (policy == std::string("transformer:w4a16-g") + group + "-v6") return QI_SCHEME_W4A16;
        if (policy == std::string("transformer:w4a4-h256-g") + group + "-v6") return QI_SCHEME_W4A4_H256;
    }
    return 0;
}

struct Pack {
    FILE *file = nullptr;
    Header header;
    std::vector<Record> records;
    std::string metadata;
};

enum : int {  // what qi_pack_* return besides 0
    PACK_IO = 20001, PACK_NOT_A_PACK = 20002, PACK_POLICY = 20003, PACK_METADATA = 20004, PACK_RECORD = 20005,
    PACK_LAYOUT = 20006, PACK_TENSOR_CHECKSUM = 20007, PACK_INVENTORY = 20008, PACK_PAYLOAD_CHECKSUM = 20009,
    PACK_ARGUMENT = 20010,
};

inline int open_pack(const char *path, Pack *pack) {
    pack->file = fopen(path, "rb");
    if (pack->file == nullptr) return PACK_IO;
    if (!read_exact(pack->file, &pack->header, HEADER_BYTES, 0)) return PACK_IO;
    const Header &h = pack->header;
    if (memcmp(h.magic, MAGIC, 8) != 0 || h.header_bytes != HEADER_BYTES || h.tensor_count == 0 || h.tensor_count > (1u << 20))
        return PACK_NOT_A_PACK;
    const uint64_t directory_end = h.directory_offset + RECORD_BYTES * h.tensor_count;
    if (h.directory_offset < HEADER_BYTES || directory_end > h.data_offset || h.data_offset > h.file_bytes) return PACK_LAYOUT;
    if (h.metadata_bytes != 0 && (h.metadata_offset < directory_end || h.metadata_offset + h.metadata_bytes > h.data_offset))
        return PACK_METADATA;
    pack->records.resize(h.tensor_count);
    if (!read_exact(pack->file, pack->records.data(), RECORD_BYTES * h.tensor_count, h.directory_offset)) return PACK_IO;
    pack->metadata.resize(h.metadata_bytes);
    if (h.metadata_bytes != 0 && !read_exact(pack->file, &pack->metadata[0], h.metadata_bytes, h.metadata_offset)) return PACK_IO;
    return 0;
}

// int4_pack.cplus:746-850. expected_tensors / expected_matrices < 0: any count (the reference fixes 297 and 224).
inline int verify_pack(const char *path, int expected_tensors, int expected_matrices) {
    Pack pack;
    int status = open_pack(path, &pack);
    struct Closer { FILE *f; ~Closer() { if (f) fclose(f); } } closer{pack.file};
    if (status != 0) return status;
    const Header &h = pack.header;
    if (expected_tensors >= 0 && h.tensor_count != static_cast<uint32_t>(expected_tensors)) return PACK_NOT_A_PACK;
    const uint32_t quantised = policy_scheme(fixed_string(h.policy, 32));
    if (quantised == 0) return PACK_POLICY;
    const uint64_t directory_end = h.directory_offset + RECORD_BYTES * h.tensor_count;
    if (h.metadata_offset < directory_end || h.metadata_offset + h.metadata_bytes > h.data_offset) return PACK_METADATA;
    if (hash_update(FNV_OFFSET, reinterpret_cast<const uint8_t *>(pack.metadata.data()), pack.metadata.size()) != h.metadata_checksum)
        return PACK_METADATA;
    std::vector<uint8_t> bytes;
    uint64_t cursor = h.data_offset;
    int matrices = 0;
    for (const Record &record : pack.records) {
        if (record.scheme == quantised) {
            ++matrices;
            const uint64_t outputs = record.dimensions[0], inputs = record.dimensions[1], group = record.group_size;
            const uint64_t groups = group == 0 ? 0 : outputs * (inputs / group);
            if (group == 0 || inputs % group != 0 || record.weights_length != outputs * inputs / 2 ||
                record.scales_length != groups * 2 ||
                record.zeros_length != (quantised == QI_SCHEME_W4A16 ? groups * 2 : 0))
                return PACK_RECORD;
        } else if (record.scheme != SCHEME_BF16 && record.scheme != SCHEME_FP16) {
            return PACK_RECORD;
        }
        const uint64_t parts[6] = {record.weights_offset, record.weights_length, record.scales_offset,
                                   record.scales_length, record.zeros_offset, record.zeros_length};
        uint64_t tensor_hash = FNV_OFFSET;
        for (int part = 0; part < 6; part += 2) {
            const uint64_t offset = parts[part], length = parts[part + 1];
            if (length == 0) continue;
            if (offset % TENSOR_ALIGNMENT != 0 || offset < cursor || offset + length > h.file_bytes) return PACK_LAYOUT;
            bytes.resize(length);
            if (!read_exact(pack.file, bytes.data(), length, offset)) return PACK_IO;
            tensor_hash = hash_update(tensor_hash, bytes.data(), length);
            cursor = offset + length;
        }
        if (tensor_hash != record.tensor_checksum) return PACK_TENSOR_CHECKSUM;
    }
    if ((expected_matrices >= 0 && matrices != expected_matrices) || align_up(cursor, TENSOR_ALIGNMENT) != h.file_bytes)
        return PACK_INVENTORY;
    bytes.resize(IO_CHUNK);
    uint64_t payload = FNV_OFFSET;
    for (uint64_t position = h.data_offset; position < h.file_bytes;) {
        const uint64_t remaining = h.file_bytes - position;
        const size_t amount = remaining < IO_CHUNK ? static_cast<size_t>(remaining) : IO_CHUNK;
        if (!read_exact(pack.file, bytes.data(), amount, position)) return PACK_IO;
        payload = hash_update(payload, bytes.data(), amount);
        position += amount;
    }
    return payload == h.payload_checksum ? 0 : PACK_PAYLOAD_CHECKSUM;
}

// Writes tensors that are already in their stored form. Matrices of the pack's quantised scheme get the record
// fields plan_record gives them; everything else is stored as given (scheme 0 or 1). Written to <path>.tmp,
// verified, then renamed (int4_pack.cplus:607-677).
inline int write_pack(const char *path, const char *policy, const char *metadata, const qi_pack_tensor *tensors, int count) {
    if (path == nullptr || policy == nullptr || tensors == nullptr || count <= 0) return PACK_ARGUMENT;
    const uint32_t quantised = policy_scheme(policy);
    if (quantised == 0) return PACK_POLICY;
    const std::string text = metadata != nullptr ? metadata : "";
    Header header;
    memset(&header, 0, sizeof(header));
    memcpy(header.magic, MAGIC, 8);
    header.version = 1;
    header.header_bytes = HEADER_BYTES;
    header.tensor_count = static_cast<uint32_t>(count);
    header.directory_offset = HEADER_BYTES;
    const uint64_t directory_end = header.directory_offset + RECORD_BYTES * count;
    header.data_offset = align_up(directory_end + text.size(), 4096);
    if (!fixed_text(header.policy, 32, policy)) return PACK_POLICY;
    std::vector<Record> records(count);
    uint64_t cursor = header.data_offset;
    for (int i = 0; i < count; ++i) {
        const qi_pack_tensor &t = tensors[i];
        Record &r = records[i];
        memset(&r, 0, sizeof(r));
        if (t.name == nullptr || !fixed_text(r.name, 128, t.name) || t.weights == nullptr || t.rank > 4) return PACK_ARGUMENT;
        r.scheme = t.scheme;
        r.rank = t.rank;
        r.elements = 1;
        for (uint32_t d = 0; d < 4; ++d) {
            r.dimensions[d] = d < t.rank ? t.dimensions[d] : 0;
            if (d < t.rank) r.elements *= t.dimensions[d];
        }
        r.weights_length = t.weights_length;
        if (t.scheme == quantised) {
            const uint64_t outputs = t.dimensions[0], inputs = t.dimensions[1], group = t.group_size;
            if (t.rank != 2 || group < 32 || group > 256 || group % 2 != 0 || 256 % group != 0 || inputs % 256 != 0)
                return PACK_RECORD;  // options_valid, int4_pack.cplus:520-525, and the K % 256 rule of :584
            const uint64_t groups = outputs * (inputs / group);
            r.group_axis = 1;
            r.group_size = t.group_size;
            r.scale_type = TYPE_F16;
            r.zero_type = quantised == QI_SCHEME_W4A16 ? TYPE_F16 : TYPE_NONE;
            r.scales_length = groups * 2;
            r.zeros_length = quantised == QI_SCHEME_W4A16 ? groups * 2 : 0;
            if (t.weights_length != outputs * inputs / 2 || t.scales == nullptr || t.scales_length != r.scales_length ||
                (r.zeros_length != 0 && (t.zeros == nullptr || t.zeros_length != r.zeros_length)))
                return PACK_RECORD;
        } else if (t.scheme != SCHEME_BF16 && t.scheme != SCHEME_FP16) {
            return PACK_RECORD;
        }
        cursor = align_up(cursor, TENSOR_ALIGNMENT);
        r.weights_offset = cursor;
        cursor += r.weights_length;
        if (r.scales_length != 0) {
            cursor = align_up(cursor, TENSOR_ALIGNMENT);
            r.scales_offset = cursor;
            cursor += r.scales_length;
        }
        if (r.zeros_length != 0) {
            cursor = align_up(cursor, TENSOR_ALIGNMENT);
            r.zeros_offset = cursor;
            cursor += r.zeros_length;
        }
        uint64_t hash = hash_update(FNV_OFFSET, static_cast<const uint8_t *>(t.weights), r.weights_length);
        if (r.scales_length != 0) hash = hash_update(hash, static_cast<const uint8_t *>(t.scales), r.scales_length);
        if (r.zeros_length != 0) hash = hash_update(hash, static_cast<const uint8_t *>(t.zeros), r.zeros_length);
        r.tensor_checksum = hash;
    }
    header.file_bytes = align_up(cursor, TENSOR_ALIGNMENT);
    header.metadata_offset = directory_end;
    header.metadata_bytes = static_cast<uint32_t>(text.size());
    header.metadata_version = METADATA_VERSION;
    header.metadata_checksum = hash_update(FNV_OFFSET, reinterpret_cast<const uint8_t *>(text.data()), text.size());

    // the data section is built in memory: its checksum covers the padding between regions too
    std::vector<uint8_t> data(header.file_bytes - header.data_offset, 0);
    for (int i = 0; i < count; ++i) {
        const Record &r = records[i];
        memcpy(&data[r.weights_offset - header.data_offset], tensors[i].weights, r.weights_length);
        if (r.scales_length != 0) memcpy(&data[r.scales_offset - header.data_offset], tensors[i].scales, r.scales_length);
        if (r.zeros_length != 0) memcpy(&data[r.zeros_offset - header.data_offset], tensors[i].zeros, r.zeros_length);
    }
    header.payload_checksum = hash_update(FNV_OFFSET, data.data(), data.size());

    const std::string temporary = std::string(path) + ".tmp";
    FILE *file = fopen(temporary.c_str(), "wb");
    if (file == nullptr) return PACK_IO;
    std::vector<uint8_t> front(header.data_offset, 0);
    memcpy(&front[0], &header, HEADER_BYTES);
    memcpy(&front[header.directory_offset], records.data(), RECORD_BYTES * count);
    memcpy(&front[directory_end], text.data(), text.size());
    bool ok = write_exact(file, front.data(), front.size(), 0) && write_exact(file, data.data(), data.size(), header.data_offset);
    ok = ok && fflush(file) == 0 && fsync(fileno(file)) == 0;
    ok = (fclose(file) == 0) && ok;
    if (!ok || verify_pack(temporary.c_str(), -1, -1) != 0) {
        remove(temporary.c_str());
        return PACK_IO;
    }
    if (rename(temporary.c_str(), path) != 0) {
        remove(temporary.c_str());
        return PACK_IO;
    }
    return 0;
}

}  // namespace pack
}  // namespace qi

extern "C" {

int qi_pack_open(const char *path, void **pack) {
    if (path == nullptr || pack == nullptr) return qi::pack::PACK_ARGUMENT;
    qi::pack::Pack *opened = new qi::pack::Pack();
    const int status = qi::pack::open_pack(path, opened);
    if (status != 0) {
        if (opened->file != nullptr) fclose(opened->file);
        delete opened;
        return status;
    }
    *pack = opened;
    return 0;
}

int qi_pack_close(void *pack) {
    if (pack == nullptr) return qi::pack::PACK_ARGUMENT;
    qi::pack::Pack *opened = static_cast<qi::pack::Pack *>(pack);
    if (opened->file != nullptr) fclose(opened->file);
    delete opened;
    return 0;
}

int qi_pack_info(void *pack, qi_pack_header_info *info) {
    if (pack == nullptr || info == nullptr) return qi::pack::PACK_ARGUMENT;
    const qi::pack::Header &h = static_cast<qi::pack::Pack *>(pack)->header;
    memset(info, 0, sizeof(*info));
    memcpy(info->policy, h.policy, 32);
    info->scheme = qi::pack::policy_scheme(qi::pack::fixed_string(h.policy, 32));
    info->tensor_count = h.tensor_count;
    info->data_offset = h.data_offset;
    info->file_bytes = h.file_bytes;
    info->payload_checksum = h.payload_checksum;
    return 0;
}

int qi_pack_record(void *pack, int index, qi_pack_record_info *info) {
    if (pack == nullptr || info == nullptr) return qi::pack::PACK_ARGUMENT;
    const qi::pack::Pack *opened = static_cast<const qi::pack::Pack *>(pack);
    if (index < 0 || static_cast<size_t>(index) >= opened->records.size()) return qi::pack::PACK_ARGUMENT;
    const qi::pack::Record &r = opened->records[index];
    memset(info, 0, sizeof(*info));
    memcpy(info->name, r.name, 128);
    info->scheme = r.scheme;
    info->rank = r.rank;
    memcpy(info->dimensions, r.dimensions, sizeof(r.dimensions));
    info->group_size = r.group_size;
    info->weights_offset = r.weights_offset, info->weights_length = r.weights_length;
    info->scales_offset = r.scales_offset, info->scales_length = r.scales_length;
    info->zeros_offset = r.zeros_offset, info->zeros_length = r.zeros_length;
    info->tensor_checksum = r.tensor_checksum;
    return 0;
}

int qi_pack_metadata(void *pack, const char *key, char *value, size_t capacity) {
    if (pack == nullptr || key == nullptr || value == nullptr || capacity == 0) return qi::pack::PACK_ARGUMENT;
    const std::string &text = static_cast<const qi::pack::Pack *>(pack)->metadata;
    const std::string wanted = std::string(key) + "=";
    size_t line = 0;
    while (line < text.size()) {  // key=value lines, pack_info.cplus:100-140
        size_t end = text.find('\n', line);
        if (end == std::string::npos) end = text.size();
        if (text.compare(line, wanted.size(), wanted) == 0) {
            const std::string found = text.substr(line + wanted.size(), end - line - wanted.size());
            if (found.size() + 1 > capacity) return qi::pack::PACK_ARGUMENT;
            memcpy(value, found.c_str(), found.size() + 1);
            return 0;
        }
        line = end + 1;
    }
    return qi::pack::PACK_METADATA;
}

int qi_pack_read(void *pack, uint64_t offset, uint64_t bytes, void *out) {
    if (pack == nullptr || out == nullptr) return qi::pack::PACK_ARGUMENT;
    qi::pack::Pack *opened = static_cast<qi::pack::Pack *>(pack);
    if (offset + bytes > opened->header.file_bytes) return qi::pack::PACK_LAYOUT;
    return qi::pack::read_exact(opened->file, out, bytes, offset) ? 0 : qi::pack::PACK_IO;
}

int qi_pack_linear(void *pack, int index, const void *device_data, qi_packed_linear *linear) {
    if (pack == nullptr || linear == nullptr || device_data == nullptr) return qi::pack::PACK_ARGUMENT;
    const qi::pack::Pack *opened = static_cast<const qi::pack::Pack *>(pack);
    if (index < 0 || static_cast<size_t>(index) >= opened->records.size()) return qi::pack::PACK_ARGUMENT;
    const qi::pack::Record &r = opened->records[index];
    if ((r.scheme != QI_SCHEME_W4A16 && r.scheme != QI_SCHEME_W4A4_H256) || r.rank != 2) return qi::pack::PACK_RECORD;
    const char *base = static_cast<const char *>(device_data) - opened->header.data_offset;  // transformer.cplus:569-572
    memset(linear, 0, sizeof(*linear));
    linear->scheme = r.scheme;
    linear->group_size = r.group_size;
    linear->n = static_cast<int>(r.dimensions[0]);
    linear->k = static_cast<int>(r.dimensions[1]);
    linear->weights = base + r.weights_offset;
    linear->scales = base + r.scales_offset;
    linear->zeros = r.zeros_length != 0 ? base + r.zeros_offset : nullptr;
    return 0;
}

int qi_pack_verify_ex(const char *path, int expected_tensors, int expected_matrices) {
    if (path == nullptr) return qi::pack::PACK_ARGUMENT;
    return qi::pack::verify_pack(path, expected_tensors, expected_matrices);
}

int qi_pack_verify(const char *path) { return qi_pack_verify_ex(path, 297, 224); }  // int4_pack.cplus:39, :836

int qi_pack_write(const char *path, const char *policy, const char *metadata, const qi_pack_tensor *tensors, int count) {
    return qi::pack::write_pack(path, policy, metadata, tensors, count);
}

}  // extern "C"
