// The header of a safetensors file, read and checked on the host.
//
// Layout: an 8-byte little-endian header length, a JSON object {name: {dtype, shape, data_offsets}} ("__metadata__"
// is skipped), then the payload; a tensor lies at 8 + header length + begin. The checks are those of the reference's
// readers (ignition/src/hyperion_ignition/compiler/weights.py:45-79; helios/crates/helios-hal/src/weights_plan.rs:52-90):
// the header fits the file and 64 MiB, every range lies inside the payload and holds exactly shape x element size
// bytes, ranges do not overlap, no name comes twice.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace hb {

struct TensorRecord {
    std::string name;
    std::string dtype;           // the container's name for it: BF16, F32, I32, ...
    std::vector<int64_t> shape;
    int64_t begin, end;          // offsets inside the payload
};

struct TensorTable {
    int64_t payload_start = 0;   // 8 + header length
    int64_t payload_bytes = 0;
    std::vector<TensorRecord> tensors;  // in the header's order
};

// Throws Failure{BAD_FILE, text} (the text does not name the file).
TensorTable read_safetensors_header(const std::string& path);

// Bytes per element of a container dtype, 0 for one this reader does not know.
int safetensors_element_size(const std::string& dtype);

}  // namespace hb
