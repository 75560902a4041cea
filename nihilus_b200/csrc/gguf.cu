// GGUF reader in front of the weight upload: maps a model file, walks its header the way the reference's parser does
// (include/nihilus-incl/infra/model_parser.hpp:635-671 header and key/value table, :855-880 tensor table, :890-940
// data placement) and hands Q8_0 tensors to nhb_weight_upload_q8_0 straight from the mapping.  Host code only.
//
// File layout (little endian): u32 magic 'GGUF', u32 version, u64 tensor_count, u64 kv_count; kv_count x { string key,
// u32 type, value }; tensor_count x { string name, u32 n_dims, u64 dims[n_dims], u32 type, u64 offset }; tensor data.
// Like the reference, the data section is located from the END of the file (file size - the largest tensor end) and
// each tensor's relative offset is rounded up to the file's alignment; unlike the reference, every length is checked
// against the mapping before it is used.
#include "internal.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <map>
#include <string>
#include <vector>

struct nhb_gguf {
	int fd				= -1;
	const uint8_t* base = nullptr;
	uint64_t size		= 0;
	uint32_t version	= 0;
	uint64_t alignment	= 32;// general.alignment when present
	uint64_t data_start = 0;
	struct tensor {
		std::string name;
		uint32_t n_dims = 0;
		uint64_t dims[4] = { 1, 1, 1, 1 };
		uint32_t type	= 0;
		uint64_t offset = 0;// relative to data_start, as stored
		uint64_t bytes	= 0;
	};
	std::vector<tensor> tensors;
	std::map<std::string, size_t> by_name;
	// scalar key/values kept for the caller (numbers as double, strings verbatim)
	std::map<std::string, double> numbers;
	std::map<std::string, std::string> strings;
};

namespace {

	thread_local std::string g_open_error;

	constexpr uint32_t GGUF_MAGIC		 = 0x46554747;// model_parser.hpp:639
	constexpr uint64_t MAX_TENSOR_COUNT	 = 100000;// :646
	constexpr uint64_t MAX_KV_COUNT		 = 10000;// :647
	constexpr uint32_t MAX_DIMENSIONS	 = 4;// :862
	constexpr uint64_t MAX_DIM_SIZE		 = 1ull << 32;// :869
	constexpr uint64_t MAX_STRING_LENGTH = 1ull << 30;

	enum value_type : uint32_t { T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STRING, T_ARRAY, T_U64, T_I64, T_F64 };// :31-46

	struct cursor {
		const uint8_t* p;
		const uint8_t* end;
		bool ok = true;
		template<typename T> T read() {
			T v{};
			if (!ok || static_cast<uint64_t>(end - p) < sizeof(T)) {
				ok = false;
				return v;
			}
			std::memcpy(&v, p, sizeof(T));
			p += sizeof(T);
			return v;
		}
		std::string read_string() {
			const uint64_t n = read<uint64_t>();
			if (!ok || n > MAX_STRING_LENGTH || static_cast<uint64_t>(end - p) < n) {
				ok = false;
				return {};
			}
			std::string s(reinterpret_cast<const char*>(p), n);
			p += n;
			return s;
		}
		void skip(uint64_t n) {
			if (!ok || static_cast<uint64_t>(end - p) < n)
				ok = false;
			else
				p += n;
		}
	};

	uint64_t scalar_size(uint32_t t) {
		switch (t) {
			case T_U8:
			case T_I8:
			case T_BOOL:
				return 1;
			case T_U16:
			case T_I16:
				return 2;
			case T_U32:
			case T_I32:
			case T_F32:
				return 4;
			case T_U64:
			case T_I64:
			case T_F64:
				return 8;
			default:
				return 0;
		}
	}

	// reads one value; scalars and strings are recorded under `key`, arrays are walked and dropped
	bool read_value(cursor& c, uint32_t type, const std::string& key, nhb_gguf* g) {
		switch (type) {
			case T_U8:
				g->numbers[key] = c.read<uint8_t>();
				return c.ok;
			case T_I8:
				g->numbers[key] = c.read<int8_t>();
				return c.ok;
			case T_BOOL:
				g->numbers[key] = c.read<uint8_t>() != 0;
				return c.ok;
			case T_U16:
				g->numbers[key] = c.read<uint16_t>();
				return c.ok;
			case T_I16:
				g->numbers[key] = c.read<int16_t>();
				return c.ok;
			case T_U32:
				g->numbers[key] = c.read<uint32_t>();
				return c.ok;
			case T_I32:
				g->numbers[key] = c.read<int32_t>();
				return c.ok;
			case T_F32:
				g->numbers[key] = c.read<float>();
				return c.ok;
			case T_U64:
				g->numbers[key] = static_cast<double>(c.read<uint64_t>());
				return c.ok;
			case T_I64:
				g->numbers[key] = static_cast<double>(c.read<int64_t>());
				return c.ok;
			case T_F64:
				g->numbers[key] = c.read<double>();
				return c.ok;
			case T_STRING:
				g->strings[key] = c.read_string();
				return c.ok;
			case T_ARRAY: {
				const uint32_t et = c.read<uint32_t>();
				const uint64_t n  = c.read<uint64_t>();
				if (!c.ok)
					return false;
				if (et == T_STRING) {
					for (uint64_t i = 0; i < n && c.ok; ++i) {
						const uint64_t len = c.read<uint64_t>();
						if (len > MAX_STRING_LENGTH)
							c.ok = false;
						c.skip(len);
					}
				} else if (et == T_ARRAY || scalar_size(et) == 0) {
					return false;// nested arrays do not occur in model files; unknown element types cannot be skipped
				} else {
					if (n > (uint64_t(1) << 40))
						return false;
					c.skip(n * scalar_size(et));
				}
				return c.ok;
			}
			default:
				return false;
		}
	}

	// bytes per block / elements per block of the tensor types this library can size (common/config.hpp:179-201 ids)
	bool type_geometry(uint32_t type, uint64_t* type_size, uint64_t* block_size) {
		switch (type) {
			case 0:// f32
				*type_size = 4, *block_size = 1;
				return true;
			case 1:// f16
				*type_size = 2, *block_size = 1;
				return true;
			case 8:// q8_0
				*type_size = 34, *block_size = 32;
				return true;
			case 24:// i8
				*type_size = 1, *block_size = 1;
				return true;
			case 25:// i16
				*type_size = 2, *block_size = 1;
				return true;
			case 26:// i32
				*type_size = 4, *block_size = 1;
				return true;
			case 27:// i64
			case 28:// f64
				*type_size = 8, *block_size = 1;
				return true;
			default:
				return false;
		}
	}

	uint64_t align_offset(uint64_t offset, uint64_t alignment) {// model_parser.hpp:890-893
		alignment = alignment == 0 ? 1 : alignment;
		return offset + (alignment - (offset % alignment)) % alignment;
	}

	int open_fail(nhb_gguf* g, int code, const std::string& msg) {
		g_open_error = msg;
		if (g) {
			if (g->base)
				munmap(const_cast<uint8_t*>(g->base), g->size);
			if (g->fd >= 0)
				close(g->fd);
			delete g;
		}
		return code;
	}

}

extern "C" {

const char* nhb_gguf_last_error(void) {
	return g_open_error.c_str();
}

int nhb_gguf_open(const char* path, nhb_gguf** out) {
	if (!path || !out)
		return open_fail(nullptr, NHB_ERR_ARG, "nhb_gguf_open: null argument");
	*out		= nullptr;
	nhb_gguf* g = new nhb_gguf();
	g->fd		= open(path, O_RDONLY);
	if (g->fd < 0)
		return open_fail(g, NHB_ERR_ARG, std::string("cannot open ") + path);
	struct stat st;
	if (fstat(g->fd, &st) != 0 || st.st_size < 24)
		return open_fail(g, NHB_ERR_ARG, "file too small for a GGUF header");
	g->size		= static_cast<uint64_t>(st.st_size);
	void* m		= mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
	if (m == MAP_FAILED)
		return open_fail(g, NHB_ERR_NOMEM, "mmap failed");
	g->base = static_cast<const uint8_t*>(m);
	cursor c{ g->base, g->base + g->size };
	if (c.read<uint32_t>() != GGUF_MAGIC)
		return open_fail(g, NHB_ERR_ARG, "not a GGUF file (magic)");
	g->version				= c.read<uint32_t>();
	const uint64_t n_tensor = c.read<uint64_t>();
	const uint64_t n_kv		= c.read<uint64_t>();
	if (!c.ok || n_tensor > MAX_TENSOR_COUNT)
		return open_fail(g, NHB_ERR_ARG, "tensor count exceeds the maximum");
	if (n_kv > MAX_KV_COUNT)
		return open_fail(g, NHB_ERR_ARG, "metadata count exceeds the maximum");
	for (uint64_t i = 0; i < n_kv; ++i) {
		const std::string key = c.read_string();
		const uint32_t type	  = c.read<uint32_t>();
		if (!c.ok || !read_value(c, type, key, g))
			return open_fail(g, NHB_ERR_ARG, "truncated or malformed metadata near key '" + key + "'");
	}
	auto al = g->numbers.find("general.alignment");
	if (al != g->numbers.end() && al->second >= 1)
		g->alignment = static_cast<uint64_t>(al->second);
	uint64_t max_end = 0;
	g->tensors.reserve(n_tensor);
	for (uint64_t i = 0; i < n_tensor; ++i) {
		nhb_gguf::tensor t;
		t.name	 = c.read_string();
		t.n_dims = c.read<uint32_t>();
		if (!c.ok || t.n_dims > MAX_DIMENSIONS)
			return open_fail(g, NHB_ERR_ARG, "tensor '" + t.name + "': more than 4 dimensions or truncated table");
		for (uint32_t d = 0; d < t.n_dims; ++d) {
			t.dims[d] = c.read<uint64_t>();
			if (t.dims[d] > MAX_DIM_SIZE)
				return open_fail(g, NHB_ERR_ARG, "tensor '" + t.name + "': dimension too large");
		}
		t.type	 = c.read<uint32_t>();
		t.offset = c.read<uint64_t>();
		if (!c.ok)
			return open_fail(g, NHB_ERR_ARG, "truncated tensor table");
		uint64_t ts = 0, bs = 0;
		if (!type_geometry(t.type, &ts, &bs))
			return open_fail(g, NHB_ERR_UNSUPPORTED, "tensor '" + t.name + "': type " + std::to_string(t.type) + " cannot be sized by this reader");
		if (t.dims[0] % bs != 0)
			return open_fail(g, NHB_ERR_ARG, "tensor '" + t.name + "': row length is not a multiple of its block size");
		// common/type_traits.hpp:38-60 for contiguous tensors: blocks per row x type size x rows
		// (each factor may be up to 2^32: the product is formed with overflow checks, a wrapped size would pass every
		// "inside the file" test below)
		uint64_t bytes = t.dims[0] / bs;
		bool wrapped   = __builtin_mul_overflow(bytes, ts, &bytes);
		for (int d = 1; d < 4; ++d)
			wrapped = wrapped || __builtin_mul_overflow(bytes, t.dims[d], &bytes);
		if (wrapped)
			return open_fail(g, NHB_ERR_ARG, "tensor '" + t.name + "': size does not fit 64 bits");
		t.bytes = bytes;
		if (t.offset > g->size || t.bytes > g->size)
			return open_fail(g, NHB_ERR_ARG, "tensor '" + t.name + "': data outside the file");
		max_end = std::max(max_end, t.offset + t.bytes);
		g->by_name[t.name] = g->tensors.size();
		g->tensors.push_back(std::move(t));
	}
	const uint64_t table_end = static_cast<uint64_t>(c.p - g->base);
	if (max_end > g->size || g->size - max_end < table_end)
		return open_fail(g, NHB_ERR_ARG, "tensor data overlaps the header or runs past the end of the file");
	g->data_start = g->size - max_end;// model_parser.hpp:927
	for (const auto& t: g->tensors)
		if (align_offset(t.offset, g->alignment) + t.bytes > max_end)
			return open_fail(g, NHB_ERR_ARG, "tensor '" + t.name + "': aligned offset runs past the end of the data section");
	*out = g;
	return NHB_OK;
}

int nhb_gguf_close(nhb_gguf* g) {
	if (!g)
		return NHB_OK;
	munmap(const_cast<uint8_t*>(g->base), g->size);
	close(g->fd);
	delete g;
	return NHB_OK;
}

int64_t nhb_gguf_tensor_count(const nhb_gguf* g) {
	return g ? static_cast<int64_t>(g->tensors.size()) : -1;
}

int64_t nhb_gguf_find(const nhb_gguf* g, const char* name) {
	if (!g || !name)
		return -1;
	auto it = g->by_name.find(name);
	return it == g->by_name.end() ? -1 : static_cast<int64_t>(it->second);
}

int nhb_gguf_tensor_get(const nhb_gguf* g, int64_t index, nhb_gguf_tensor* out) {
	if (!g || !out || index < 0 || index >= static_cast<int64_t>(g->tensors.size()))
		return NHB_ERR_ARG;
	const auto& t = g->tensors[static_cast<size_t>(index)];
	out->name	  = t.name.c_str();
	out->n_dims	  = static_cast<int>(t.n_dims);
	for (int d = 0; d < 4; ++d)
		out->dims[d] = static_cast<int64_t>(t.dims[d]);
	out->type	= static_cast<int>(t.type);
	out->bytes	= static_cast<int64_t>(t.bytes);
	out->offset = static_cast<int64_t>(g->data_start + align_offset(t.offset, g->alignment));
	out->data	= g->base + out->offset;
	return NHB_OK;
}

int nhb_gguf_get_number(const nhb_gguf* g, const char* key, double* out) {
	if (!g || !key || !out)
		return NHB_ERR_ARG;
	auto it = g->numbers.find(key);
	if (it == g->numbers.end())
		return NHB_ERR_ARG;
	*out = it->second;
	return NHB_OK;
}

const char* nhb_gguf_get_string(const nhb_gguf* g, const char* key) {
	if (!g || !key)
		return nullptr;
	auto it = g->strings.find(key);
	return it == g->strings.end() ? nullptr : it->second.c_str();
}

int nhb_gguf_upload_q8_0(nhb_ctx* ctx, const nhb_gguf* g, const char* name, nhb_weight** out) {
	if (!ctx || !g || !name || !out)
		return NHB_ERR_ARG;
	*out			  = nullptr;
	const int64_t idx = nhb_gguf_find(g, name);
	if (idx < 0)
		return NHB_ERR_ARG;
	nhb_gguf_tensor t;
	nhb_gguf_tensor_get(g, idx, &t);
	if (t.type != 8 || t.n_dims > 2 || t.dims[2] != 1 || t.dims[3] != 1)
		return NHB_ERR_UNSUPPORTED;// not a Q8_0 matrix
	// GGUF stores ne0 = K (the contiguous, quantised dimension) first, ne1 = N rows
	return nhb_weight_upload_q8_0(ctx, t.data, t.dims[1], t.dims[0], out);
}

int nhb_gguf_read_f32(const nhb_gguf* g, const char* name, float* dst, int64_t count) {
	if (!g || !name || !dst || count < 0)
		return NHB_ERR_ARG;
	const int64_t idx = nhb_gguf_find(g, name);
	if (idx < 0)
		return NHB_ERR_ARG;
	nhb_gguf_tensor t;
	nhb_gguf_tensor_get(g, idx, &t);
	if (t.type != 0 || t.bytes != count * 4)
		return NHB_ERR_ARG;
	std::memcpy(dst, t.data, static_cast<size_t>(t.bytes));
	return NHB_OK;
}
}
