/*
 * NVFP4 tensors in the weights section of a model artifact: parse, validate,
 * stage into one device block, register.
 *
 * mimfer's loader reads the section's tensor index and stages every tensor into
 * the weight arena (src/model/tensor_registry.c:372-560), but accepts bf16
 * entries only: an MM_DT_FP4E2M1 entry is rejected with MM_ERR_UNSUPPORTED
 * (tensor_registry.c:468-474), so its planner never sees an fp4 tensor
 * (src/plan/plan.c:204-220 branches on is_fp4).  This file is that missing
 * branch.  Index layout and validation gates follow the reference
 * (src/model/tensor_registry.h:86-120):
 *
 *   u32 version (1), u32 flags (0), u32 n_tensors
 *   per tensor: u16 name_len (1..48, NUL included), name, u32 rows, u32 cols,
 *               u8 dtype, u8 pad[3], u64 offset, u64 nbytes
 *   tensor bytes (offsets are relative to the start of the section payload)
 *
 * A bf16 entry carries rows*cols*2 bytes.  An fp4 entry carries, back to back,
 *   payload  rows * cols/2 bytes   (low nibble = even column, tensor.h:17-19)
 *   scales   rows * cols/16 bytes  (e4m3, one per 16 columns)
 *   global   4 bytes               (fp32, little endian)
 * so nbytes = rows*cols*9/16 + 4 and cols must be a multiple of 16.
 *
 * The gates that tie the index to a model shape (count and order against the
 * canonical tensor list, tensor_registry.c:418-437 and :513-525) belong to the
 * model section and are not repeated here.
 *
 * Staging follows the arena discipline of the reference (alloc.h:4-29): the
 * caller owns ONE device block, sized by mm_f4_weights_arena_bytes; tensors are
 * bump-placed in index order on 256-byte boundaries (tensor_registry.c:223),
 * payload first, then scales.  Tensors adjacent in the index are therefore
 * adjacent in memory in a fixed order, which is what the fused gate/up kernel
 * needs.  Nothing is allocated on the device here.
 */
#include "../core/core.h"
#include <stdlib.h>
#include <string.h>

#define WT_VERSION   1u
#define WT_MAX       4096u            /* MM_MAX_TENSORS, include/mimfer/engine.h:71 */
#define WT_ALIGN     256u

static uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static uint32_t rd32(const uint8_t *p)
{
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}
static uint64_t rd64(const uint8_t *p) { return (uint64_t)rd32(p) | ((uint64_t)rd32(p + 4) << 32); }

uint64_t mm_f4_tensor_bytes(uint32_t rows, uint32_t cols)
{
    return (uint64_t)rows * cols / 2u + (uint64_t)rows * cols / 16u + 4u;
}

mm_status mm_f4_weights_parse(const uint8_t *data, size_t len, mm_f4_went *ents, uint32_t cap,
                              uint32_t *n_out)
{
    MM_REQUIRE(data && n_out, MM_ERR_STATE);
    *n_out = 0;
    if (len < 12) {
        MM_LOGE("weights: payload %zu bytes < 12-byte index header", len);
        return MM_ERR_CORRUPT;
    }
    if (rd32(data) != WT_VERSION || rd32(data + 4) != 0) {
        MM_LOGE("weights: index version %u flags %u (this build reads version %u, flags 0)",
                rd32(data), rd32(data + 4), WT_VERSION);
        return MM_ERR_CORRUPT;
    }
    uint32_t n = rd32(data + 8);
    if (n > WT_MAX) {
        MM_LOGE("weights: n_tensors %u > %u", n, WT_MAX);
        return MM_ERR_CORRUPT;
    }
    if (ents && n > cap)
        return MM_ERR_CAPACITY;
    size_t p = 12;
    /* first pass: the index itself (its end bounds the tensor offsets) */
    size_t q = p;
    for (uint32_t i = 0; i < n; i++) {
        if (q + 2 > len)
            goto truncated;
        uint16_t nl = rd16(data + q);
        if (nl < 1 || nl > 48) {
            MM_LOGE("weights: entry %u: bad name_len %u (1..48)", i, nl);
            return MM_ERR_CORRUPT;
        }
        if (q + 2 + (size_t)nl + 28 > len)
            goto truncated;
        q += 2 + (size_t)nl + 28;
    }
    const size_t index_end = q;
    for (uint32_t i = 0; i < n; i++) {
        mm_f4_went e;
        memset(&e, 0, sizeof e);
        uint16_t nl = rd16(data + p);
        p += 2;
        if (data[p + nl - 1] != 0) {
            MM_LOGE("weights: entry %u: name not NUL-terminated", i);
            return MM_ERR_CORRUPT;
        }
        memcpy(e.name, data + p, nl);
        p += nl;
        e.rows = rd32(data + p);
        e.cols = rd32(data + p + 4);
        e.dtype = data[p + 8];
        e.off = rd64(data + p + 12);
        e.nbytes = rd64(data + p + 20);
        p += 28;
        uint64_t want;
        if (e.dtype == MM_DT_FP4E2M1) {
            if (e.cols % 16 != 0 || e.rows == 0 || e.cols == 0) {
                MM_LOGE("weights: entry %u (\"%s\"): fp4 tensor %u x %u needs cols %% 16 == 0", i,
                        e.name, e.rows, e.cols);
                return MM_ERR_SHAPE;
            }
            want = mm_f4_tensor_bytes(e.rows, e.cols);
        } else if (e.dtype == MM_DT_BF16) {
            want = (uint64_t)e.rows * e.cols * 2u;
        } else {
            MM_LOGE("weights: entry %u (\"%s\"): dtype %u is neither bf16 nor fp4", i, e.name, e.dtype);
            return MM_ERR_UNSUPPORTED;
        }
        if (e.nbytes != want) {
            MM_LOGE("weights: entry %u (\"%s\"): nbytes %llu != %llu for %u x %u", i, e.name,
                    (unsigned long long)e.nbytes, (unsigned long long)want, e.rows, e.cols);
            return MM_ERR_CORRUPT;
        }
        if (e.off < index_end || e.off > len || e.nbytes > len - e.off) {
            MM_LOGE("weights: entry %u (\"%s\"): bytes [%llu..+%llu) outside the %zu-byte payload "
                    "(index ends at %zu)", i, e.name, (unsigned long long)e.off,
                    (unsigned long long)e.nbytes, len, index_end);
            return MM_ERR_CORRUPT;
        }
        if (ents)
            ents[i] = e;
    }
    *n_out = n;
    return MM_OK;
truncated:
    MM_LOGE("weights: index truncated (%zu bytes)", len);
    return MM_ERR_CORRUPT;
}

static size_t slot(size_t v) { return mmb_align_up(v, WT_ALIGN); }

size_t mm_f4_weights_arena_bytes(const mm_f4_went *ents, uint32_t n)
{
    size_t total = 0;
    for (uint32_t i = 0; ents && i < n; i++) {
        if (ents[i].dtype == MM_DT_FP4E2M1)
            total += slot((size_t)ents[i].rows * ents[i].cols / 2u) +
                     slot((size_t)ents[i].rows * ents[i].cols / 16u);
        else
            total += slot((size_t)ents[i].nbytes);
    }
    return total;
}

/* ------------------------------------------------------------- registry */
typedef struct wt_view {
    char        name[48];
    int         is_fp4;
    mm_wt       w;          /* fp4: payload, scales, rows, cols          */
    float       gs;         /* fp4: global scale                          */
    const void *data;       /* bf16: device pointer                       */
    size_t      bytes;
    uint32_t    rows, cols;
} wt_view;

struct mm_f4_wreg {
    wt_view *v;
    uint32_t n;
    size_t   used;          /* bytes of the arena taken */
};

mm_status mm_f4_weights_stage(const uint8_t *data, size_t len, void *arena_dev, size_t arena_bytes,
                              mm_f4_wreg **out)
{
    MM_REQUIRE(data && arena_dev && out, MM_ERR_STATE);
    MM_REQUIRE(((uintptr_t)arena_dev & (WT_ALIGN - 1u)) == 0, MM_ERR_SHAPE);
    *out = NULL;
    uint32_t n = 0;
    mm_status st = mm_f4_weights_parse(data, len, NULL, 0, &n);
    if (st != MM_OK)
        return st;
    mm_f4_went *ents = (mm_f4_went *)calloc(n ? n : 1, sizeof *ents);
    mm_f4_wreg *reg = (mm_f4_wreg *)calloc(1, sizeof *reg);
    wt_view *views = (wt_view *)calloc(n ? n : 1, sizeof *views);
    if (!ents || !reg || !views) {
        st = MM_ERR_NOMEM;
        goto fail;
    }
    st = mm_f4_weights_parse(data, len, ents, n, &n);
    if (st != MM_OK)
        goto fail;
    if (mm_f4_weights_arena_bytes(ents, n) > arena_bytes) {
        MM_LOGE("weights: %u tensors need %zu bytes, the arena holds %zu", n,
                mm_f4_weights_arena_bytes(ents, n), arena_bytes);
        st = MM_ERR_CAPACITY;
        goto fail;
    }
    for (uint32_t i = 0; i < n; i++)
        for (uint32_t j = 0; j < i; j++)
            if (strcmp(ents[i].name, ents[j].name) == 0) {
                MM_LOGE("weights: duplicate tensor name \"%s\"", ents[i].name);
                st = MM_ERR_CORRUPT;
                goto fail;
            }
    /* Everything that can be refused is refused before the first copy or
     * registration (the reference loader's "no partial state" gate,
     * src/model/tensor_registry.c:372-560): global scales and the room left in
     * the scale registry. */
    uint32_t n_fp4 = 0;
    for (uint32_t i = 0; i < n; i++) {
        const mm_f4_went *e = &ents[i];
        if (e->dtype != MM_DT_FP4E2M1)
            continue;
        size_t pb = (size_t)e->rows * e->cols / 2u, sb = (size_t)e->rows * e->cols / 16u;
        uint32_t bits = rd32(data + e->off + pb + sb);
        float gs;
        memcpy(&gs, &bits, 4);
        if (!(gs > 0.0f && gs < 3.0e38f)) {
            MM_LOGE("weights: \"%s\": global scale %g is not a positive finite number", e->name, (double)gs);
            st = MM_ERR_CORRUPT;
            goto fail;
        }
        n_fp4++;
    }
    if (n_fp4 > mm_f4_gscale_room()) {
        MM_LOGE("weights: %u NVFP4 tensors, the global-scale registry has room for %u", n_fp4,
                mm_f4_gscale_room());
        st = MM_ERR_CAPACITY;
        goto fail;
    }
    uint8_t *base = (uint8_t *)arena_dev;
    size_t at = 0;
    uint32_t done = 0;                      /* tensors whose scale is registered */
    for (uint32_t i = 0; i < n; i++) {
        const mm_f4_went *e = &ents[i];
        wt_view *v = &views[i];
        memcpy(v->name, e->name, sizeof v->name);
        v->rows = e->rows;
        v->cols = e->cols;
        const uint8_t *src = data + e->off;
        if (e->dtype == MM_DT_FP4E2M1) {
            size_t pb = (size_t)e->rows * e->cols / 2u, sb = (size_t)e->rows * e->cols / 16u;
            uint8_t *pay = base + at, *scl = pay + slot(pb);
            at += slot(pb) + slot(sb);
            if ((st = mm_h2d_async(pay, src, pb, MM_ST_XFER)) != MM_OK ||
                (st = mm_h2d_async(scl, src + pb, sb, MM_ST_XFER)) != MM_OK)
                goto unwind;
            uint32_t bits = rd32(src + pb + sb);
            memcpy(&v->gs, &bits, 4);
            v->is_fp4 = 1;
            v->w.data = pay;
            v->w.scale = scl;
            v->w.rows = e->rows;
            v->w.cols = e->cols;
            if ((st = mm_f4_gscale_set(scl, v->gs)) != MM_OK)
                goto unwind;
        } else {
            uint8_t *dst = base + at;
            at += slot((size_t)e->nbytes);
            if ((st = mm_h2d_async(dst, src, (size_t)e->nbytes, MM_ST_XFER)) != MM_OK)
                goto unwind;
            v->data = dst;
            v->bytes = (size_t)e->nbytes;
        }
        done = i + 1;
    }
    if ((st = mm_stream_sync(MM_ST_XFER)) != MM_OK)
        goto unwind;
    reg->v = views;
    reg->n = n;
    reg->used = at;
    free(ents);
    MM_LOGI("weights: staged %u tensors (%zu bytes of the arena)", n, at);
    *out = reg;
    return MM_OK;
unwind:
    /* copies from `data` may still be in flight and some scales are registered
     * under arena addresses the caller will reuse: wait, then take them back */
    (void)mm_stream_sync(MM_ST_XFER);
    for (uint32_t i = 0; i < done && i < n; i++)
        if (views[i].is_fp4)
            mm_f4_gscale_unset(views[i].w.scale);
    if (done < n && views[done].is_fp4 && views[done].w.scale)
        mm_f4_gscale_unset(views[done].w.scale);
fail:
    free(ents);
    free(views);
    free(reg);
    return st;
}

static const wt_view *find_view(const mm_f4_wreg *r, const char *name)
{
    for (uint32_t i = 0; r && name && i < r->n; i++)
        if (strcmp(r->v[i].name, name) == 0)
            return &r->v[i];
    return NULL;
}

uint32_t mm_f4_weights_count(const mm_f4_wreg *r) { return r ? r->n : 0; }
size_t   mm_f4_weights_used(const mm_f4_wreg *r) { return r ? r->used : 0; }

mm_status mm_f4_weights_find(const mm_f4_wreg *r, const char *name, mm_wt *w_out, float *gs_out)
{
    MM_REQUIRE(r && name && w_out, MM_ERR_STATE);
    const wt_view *v = find_view(r, name);
    if (!v)
        return MM_ERR_RANGE;
    if (!v->is_fp4)
        return MM_ERR_UNSUPPORTED;
    *w_out = v->w;
    if (gs_out)
        *gs_out = v->gs;
    return MM_OK;
}

mm_status mm_f4_weights_find_bf16(const mm_f4_wreg *r, const char *name, const void **data_out,
                                  uint32_t *rows_out, uint32_t *cols_out)
{
    MM_REQUIRE(r && name && data_out, MM_ERR_STATE);
    const wt_view *v = find_view(r, name);
    if (!v)
        return MM_ERR_RANGE;
    if (v->is_fp4)
        return MM_ERR_UNSUPPORTED;
    *data_out = v->data;
    if (rows_out) *rows_out = v->rows;
    if (cols_out) *cols_out = v->cols;
    return MM_OK;
}

void mm_f4_weights_free(mm_f4_wreg *r)
{
    if (!r)
        return;
    free(r->v);
    free(r);
}
