/* GGUF reader for the MoE feed-forward tensors (see include/tie_gguf.h).
 *
 * File layout (GGUF v2/v3, little endian): magic "GGUF", u32 version, u64 tensor count, u64 KV
 * count; KV pairs = string key, u32 value type, value (scalars, string = u64 length + bytes,
 * array = u32 element type + u64 count + elements); tensor directory = string name, u32 n_dims,
 * u64 dims[n_dims], u32 type, u64 offset relative to the data section; the data section starts at
 * the next multiple of general.alignment (default 32) after the directory.  The reference walks
 * the same structure in gguf_model_parse (gguf.c:968-1047); here every read is bounds-checked
 * against the mapping and only what the MoE path needs is kept. */
#define _GNU_SOURCE
#include "../../include/tie_gguf.h"

#include <fcntl.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

enum { VT_U8 = 0, VT_I8, VT_U16, VT_I16, VT_U32, VT_I32, VT_F32, VT_BOOL, VT_STR, VT_ARR, VT_U64, VT_I64, VT_F64, VT_COUNT };
enum { GGML_F32 = 0, GGML_F16 = 1, GGML_Q8_0 = 8, GGML_Q4_K = 12, GGML_Q6_K = 14, GGML_BF16 = 30 };

typedef struct {
	const char *name;  /* not terminated: into the mapping */
	uint64_t name_len;
	uint64_t hash;
	uint32_t vtype;	      /* KV: value type; tensor: GGMLType */
	const uint8_t *value; /* KV: first byte of the value */
	uint32_t n_dims;      /* tensor */
	uint64_t dims[4];
	uint64_t offset;
} entry;

struct tie_gguf {
	int fd;
	const uint8_t *base;
	uint64_t size;
	uint32_t version;
	uint64_t n_kv, n_tensors;
	entry *kv, *tensors;
	uint64_t data_start;
};

typedef struct {
	const uint8_t *p, *end;
	int bad;
} cursor;

static uint64_t fnv1a(const char *s, uint64_t n)
{
	uint64_t h = 1469598103934665603ull;
	for (uint64_t i = 0; i < n; i++)
		h = (h ^ (uint8_t)s[i]) * 1099511628211ull;
	return h;
}

static const uint8_t *take(cursor *c, uint64_t n)
{
	if (c->bad || (uint64_t)(c->end - c->p) < n) {
		c->bad = 1;
		return NULL;
	}
	const uint8_t *r = c->p;
	c->p += n;
	return r;
}
static uint32_t rd_u32(cursor *c)
{
	uint32_t v = 0;
	const uint8_t *p = take(c, 4);
	if (p)
		memcpy(&v, p, 4);
	return v;
}
static uint64_t rd_u64(cursor *c)
{
	uint64_t v = 0;
	const uint8_t *p = take(c, 8);
	if (p)
		memcpy(&v, p, 8);
	return v;
}
static void rd_str(cursor *c, const char **s, uint64_t *len)
{
	*len = rd_u64(c);
	*s = (const char *)take(c, *len);
}

static const uint64_t scalar_size[VT_COUNT] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};

/* Steps over one value of type vt. */
static void skip_value(cursor *c, uint32_t vt)
{
	if (vt >= VT_COUNT) {
		c->bad = 1;
	} else if (vt == VT_STR) {
		const char *s;
		uint64_t n;
		rd_str(c, &s, &n);
	} else if (vt == VT_ARR) {
		const uint32_t et = rd_u32(c);
		const uint64_t n = rd_u64(c);
		if (et >= VT_COUNT || et == VT_ARR) {
			c->bad = 1;
		} else if (et == VT_STR) {
			for (uint64_t i = 0; i < n && !c->bad; i++)
				skip_value(c, VT_STR);
		} else if (n > (uint64_t)(c->end - c->p) / scalar_size[et]) {
			c->bad = 1;
		} else {
			take(c, n * scalar_size[et]);
		}
	} else {
		take(c, scalar_size[vt]);
	}
}

static void set_err(char *err, size_t n, const char *fmt, ...)
{
	if (!err || !n)
		return;
	va_list ap;
	va_start(ap, fmt);
	vsnprintf(err, n, fmt, ap);
	va_end(ap);
}

const char *tie_gguf_strerror(int code)
{
	switch (code) {
	case TIE_GGUF_OK: return "ok";
	case TIE_GGUF_EIO: return "cannot open or map the file";
	case TIE_GGUF_EFORMAT: return "not a valid GGUF file";
	case TIE_GGUF_ENOTFOUND: return "key or tensor not found";
	case TIE_GGUF_ETYPE: return "unexpected type or shape";
	case TIE_GGUF_EINVAL: return "invalid argument";
	default: return "unknown error";
	}
}

/* Bytes of a tensor of `type` with n elements whose contiguous dimension is ne0; 0 = unsupported. */
static uint64_t tensor_bytes(uint32_t type, uint64_t n, uint64_t ne0)
{
	switch (type) {
	case GGML_F32: return n * 4;
	case GGML_F16:
	case GGML_BF16: return n * 2;
	case GGML_Q8_0: return ne0 % 32 ? 0 : n / 32 * 34;
	case GGML_Q4_K: return ne0 % 256 ? 0 : n / 256 * 144;
	case GGML_Q6_K: return ne0 % 256 ? 0 : n / 256 * 210;
	default: return 0;
	}
}

void tie_gguf_close(tie_gguf *g)
{
	if (!g)
		return;
	if (g->base)
		munmap((void *)g->base, g->size);
	if (g->fd >= 0)
		close(g->fd);
	free(g->kv);
	free(g->tensors);
	free(g);
}

int tie_gguf_open(const char *path, tie_gguf **out, char *err, size_t err_len)
{
	if (!path || !out)
		return TIE_GGUF_EINVAL;
	*out = NULL;
	tie_gguf *g = calloc(1, sizeof(*g));
	if (!g)
		return TIE_GGUF_EIO;
	g->fd = open(path, O_RDONLY);
	struct stat st;
	if (g->fd < 0 || fstat(g->fd, &st) != 0 || st.st_size < 24) {
		set_err(err, err_len, "%s: cannot open (or shorter than a GGUF header)", path);
		tie_gguf_close(g);
		return TIE_GGUF_EIO;
	}
	g->size = (uint64_t)st.st_size;
	void *m = mmap(NULL, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
	if (m == MAP_FAILED) {
		set_err(err, err_len, "%s: mmap failed", path);
		tie_gguf_close(g);
		return TIE_GGUF_EIO;
	}
	g->base = m;
	cursor c = {g->base, g->base + g->size, 0};
	const uint32_t magic = rd_u32(&c);
	g->version = rd_u32(&c);
	g->n_tensors = rd_u64(&c);
	g->n_kv = rd_u64(&c);
	if (magic != 0x46554747u || (g->version != 2 && g->version != 3)) {
		set_err(err, err_len, "%s: magic %08x version %u is not GGUF v2/v3", path, magic, g->version);
		tie_gguf_close(g);
		return TIE_GGUF_EFORMAT;
	}
	/* every entry takes at least 12 bytes of the file: bounds the counts before allocating */
	if (g->n_kv > g->size / 12 || g->n_tensors > g->size / 12) {
		set_err(err, err_len, "%s: directory counts exceed the file size", path);
		tie_gguf_close(g);
		return TIE_GGUF_EFORMAT;
	}
	g->kv = calloc(g->n_kv ? g->n_kv : 1, sizeof(entry));
	g->tensors = calloc(g->n_tensors ? g->n_tensors : 1, sizeof(entry));
	if (!g->kv || !g->tensors) {
		tie_gguf_close(g);
		return TIE_GGUF_EIO;
	}
	for (uint64_t i = 0; i < g->n_kv && !c.bad; i++) {
		entry *e = &g->kv[i];
		rd_str(&c, &e->name, &e->name_len);
		e->vtype = rd_u32(&c);
		e->value = c.p;
		skip_value(&c, e->vtype);
		if (!c.bad)
			e->hash = fnv1a(e->name, e->name_len);
	}
	for (uint64_t i = 0; i < g->n_tensors && !c.bad; i++) {
		entry *e = &g->tensors[i];
		rd_str(&c, &e->name, &e->name_len);
		e->n_dims = rd_u32(&c);
		if (e->n_dims == 0 || e->n_dims > 4) {
			c.bad = 1;
			break;
		}
		for (uint32_t d = 0; d < 4; d++)
			e->dims[d] = d < e->n_dims ? rd_u64(&c) : 1;
		e->vtype = rd_u32(&c);
		e->offset = rd_u64(&c);
		if (!c.bad)
			e->hash = fnv1a(e->name, e->name_len);
	}
	if (c.bad) {
		set_err(err, err_len, "%s: truncated or malformed metadata / tensor directory", path);
		tie_gguf_close(g);
		return TIE_GGUF_EFORMAT;
	}
	uint64_t align = 32;
	if (tie_gguf_get_u64(g, "general.alignment", &align) == TIE_GGUF_OK && (align == 0 || (align & (align - 1)))) {
		set_err(err, err_len, "%s: general.alignment %llu is not a power of two", path, (unsigned long long)align);
		tie_gguf_close(g);
		return TIE_GGUF_EFORMAT;
	}
	g->data_start = ((uint64_t)(c.p - g->base) + align - 1) / align * align;
	*out = g;
	return TIE_GGUF_OK;
}

uint32_t tie_gguf_version(const tie_gguf *g) { return g ? g->version : 0; }
uint64_t tie_gguf_tensor_count(const tie_gguf *g) { return g ? g->n_tensors : 0; }
uint64_t tie_gguf_kv_count(const tie_gguf *g) { return g ? g->n_kv : 0; }

static const entry *find(const entry *tab, uint64_t n, const char *name)
{
	const uint64_t len = strlen(name), h = fnv1a(name, len);
	for (uint64_t i = 0; i < n; i++)
		if (tab[i].hash == h && tab[i].name_len == len && memcmp(tab[i].name, name, len) == 0)
			return &tab[i];
	return NULL;
}

int tie_gguf_get_u64(const tie_gguf *g, const char *key, uint64_t *value)
{
	if (!g || !key || !value)
		return TIE_GGUF_EINVAL;
	const entry *e = find(g->kv, g->n_kv, key);
	if (!e)
		return TIE_GGUF_ENOTFOUND;
	int64_t s = 0;
	switch (e->vtype) {
	case VT_U8: case VT_BOOL: *value = e->value[0]; return TIE_GGUF_OK;
	case VT_U16: { uint16_t v; memcpy(&v, e->value, 2); *value = v; return TIE_GGUF_OK; }
	case VT_U32: { uint32_t v; memcpy(&v, e->value, 4); *value = v; return TIE_GGUF_OK; }
	case VT_U64: memcpy(value, e->value, 8); return TIE_GGUF_OK;
	case VT_I8: s = (int8_t)e->value[0]; break;
	case VT_I16: { int16_t v; memcpy(&v, e->value, 2); s = v; break; }
	case VT_I32: { int32_t v; memcpy(&v, e->value, 4); s = v; break; }
	case VT_I64: memcpy(&s, e->value, 8); break;
	default: return TIE_GGUF_ETYPE;
	}
	if (s < 0)
		return TIE_GGUF_ETYPE;
	*value = (uint64_t)s;
	return TIE_GGUF_OK;
}

int tie_gguf_get_f32(const tie_gguf *g, const char *key, float *value)
{
	if (!g || !key || !value)
		return TIE_GGUF_EINVAL;
	const entry *e = find(g->kv, g->n_kv, key);
	if (!e)
		return TIE_GGUF_ENOTFOUND;
	if (e->vtype == VT_F32) {
		memcpy(value, e->value, 4);
	} else if (e->vtype == VT_F64) {
		double d;
		memcpy(&d, e->value, 8);
		*value = (float)d;
	} else {
		return TIE_GGUF_ETYPE;
	}
	return TIE_GGUF_OK;
}

int tie_gguf_get_str(const tie_gguf *g, const char *key, char *buf, size_t buf_len)
{
	if (!g || !key || !buf || !buf_len)
		return TIE_GGUF_EINVAL;
	const entry *e = find(g->kv, g->n_kv, key);
	if (!e)
		return TIE_GGUF_ENOTFOUND;
	if (e->vtype != VT_STR)
		return TIE_GGUF_ETYPE;
	uint64_t n;
	memcpy(&n, e->value, 8);
	if (n > buf_len - 1)
		n = buf_len - 1;
	memcpy(buf, e->value + 8, n);
	buf[n] = 0;
	return TIE_GGUF_OK;
}

int tie_gguf_find_tensor(const tie_gguf *g, const char *name, tie_gguf_tensor *out)
{
	if (!g || !name || !out)
		return TIE_GGUF_EINVAL;
	const entry *e = find(g->tensors, g->n_tensors, name);
	if (!e)
		return TIE_GGUF_ENOTFOUND;
	uint64_t n = 1;
	for (uint32_t d = 0; d < e->n_dims; d++) {
		if (e->dims[d] == 0 || n > UINT64_MAX / e->dims[d])
			return TIE_GGUF_EFORMAT;
		n *= e->dims[d];
	}
	const uint64_t bytes = tensor_bytes(e->vtype, n, e->dims[0]);
	if (!bytes)
		return TIE_GGUF_ETYPE;
	if (g->data_start > g->size || e->offset > g->size - g->data_start || bytes > g->size - g->data_start - e->offset)
		return TIE_GGUF_EFORMAT;  /* the tensor does not fit in the file */
	out->data = g->base + g->data_start + e->offset;
	out->nbytes = bytes;
	out->type = e->vtype;
	out->n_dims = e->n_dims;
	memcpy(out->dims, e->dims, sizeof(out->dims));
	return TIE_GGUF_OK;
}

int tie_gguf_moe_config_read(const tie_gguf *g, tie_gguf_moe_config *cfg)
{
	if (!g || !cfg)
		return TIE_GGUF_EINVAL;
	memset(cfg, 0, sizeof(*cfg));
	int rc = tie_gguf_get_str(g, "general.architecture", cfg->arch, sizeof(cfg->arch));
	if (rc)
		return rc;
	static const char *const keys[5] = {"block_count", "embedding_length", "expert_count", "expert_used_count",
					    "expert_feed_forward_length"};
	uint32_t *const dst[5] = {&cfg->n_layers, &cfg->hidden, &cfg->n_expert, &cfg->top_k, &cfg->ffn_dim};
	char key[96];
	for (int i = 0; i < 5; i++) {
		uint64_t v;
		snprintf(key, sizeof(key), "%s.%s", cfg->arch, keys[i]);
		if ((rc = tie_gguf_get_u64(g, key, &v)) != TIE_GGUF_OK)
			return rc;
		if (v == 0 || v > 0x7fffffffu)
			return TIE_GGUF_ETYPE;
		*dst[i] = (uint32_t)v;
	}
	snprintf(key, sizeof(key), "%s.attention.layer_norm_rms_epsilon", cfg->arch);
	if (tie_gguf_get_f32(g, key, &cfg->norm_eps) != TIE_GGUF_OK)
		cfg->norm_eps = 1e-6f;
	return TIE_GGUF_OK;
}

/* A stacked expert tensor [n_expert][rows][cols], cols contiguous, Q4_K or Q6_K. */
static int expert_tensor(const tie_gguf *g, int layer, const char *which, uint64_t cols, uint64_t rows, uint64_t n_expert,
			 const void **data, int *type)
{
	char name[96];
	tie_gguf_tensor t;
	snprintf(name, sizeof(name), "blk.%d.%s.weight", layer, which);
	int rc = tie_gguf_find_tensor(g, name, &t);
	if (rc)
		return rc;
	if ((t.type != GGML_Q4_K && t.type != GGML_Q6_K) || t.n_dims != 3 || t.dims[0] != cols || t.dims[1] != rows ||
	    t.dims[2] != n_expert)
		return TIE_GGUF_ETYPE;
	*data = t.data;
	*type = (int)t.type;
	return TIE_GGUF_OK;
}

int tie_gguf_moe_layer_read(const tie_gguf *g, const tie_gguf_moe_config *cfg, int layer, tie_gguf_moe_layer *out)
{
	if (!g || !cfg || !out || layer < 0 || (uint32_t)layer >= cfg->n_layers)
		return TIE_GGUF_EINVAL;
	memset(out, 0, sizeof(*out));
	char name[96];
	tie_gguf_tensor t;
	snprintf(name, sizeof(name), "blk.%d.ffn_gate_inp.weight", layer);
	int rc = tie_gguf_find_tensor(g, name, &t);
	if (rc)
		return rc;
	if (t.type != GGML_F32 || t.n_dims != 2 || t.dims[0] != cfg->hidden || t.dims[1] != cfg->n_expert)
		return TIE_GGUF_ETYPE;
	out->router_w = t.data;
	if ((rc = expert_tensor(g, layer, "ffn_gate_exps", cfg->hidden, cfg->ffn_dim, cfg->n_expert, &out->gate_exps, &out->gate_type)) ||
	    (rc = expert_tensor(g, layer, "ffn_up_exps", cfg->hidden, cfg->ffn_dim, cfg->n_expert, &out->up_exps, &out->up_type)) ||
	    (rc = expert_tensor(g, layer, "ffn_down_exps", cfg->ffn_dim, cfg->hidden, cfg->n_expert, &out->down_exps, &out->down_type)))
		return rc;
	snprintf(name, sizeof(name), "blk.%d.ffn_norm.weight", layer);
	rc = tie_gguf_find_tensor(g, name, &t);
	if (rc == TIE_GGUF_OK) {
		if (t.type != GGML_F32 || t.n_dims != 1 || t.dims[0] != cfg->hidden)
			return TIE_GGUF_ETYPE;
		out->ffn_norm_w = t.data;
	} else if (rc != TIE_GGUF_ENOTFOUND) {
		return rc;
	}
	return TIE_GGUF_OK;
}
