/*
 * Status strings and the log sink of the NVFP4 linear library.
 * Counterpart of src/core/mimfer.c:16-60 in the mimfer tree: same status
 * vocabulary, one formatting site, messages go to stderr as
 * "<level> <file>:<line>: <text>".
 */
#include "core.h"
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

static int g_level = 1;   /* 0 errors, 1 warnings, 2 info, 3 debug */

void mm_log_set_level(int level) { g_level = level < 0 ? 0 : (level > 3 ? 3 : level); }

const char *mm_status_str(mm_status s)
{
    static const char *const names[MM_ERR_LAST] = {
        "ok", "out of memory", "i/o failure", "checksum or magic mismatch",
        "bad shape or stride", "cuda runtime failure", "device not the target profile",
        "unsupported on this build", "scalar out of range", "bad object state",
        "resource held by another owner", "wait exceeded its budget",
        "pool exhausted", "end of input" };
    return ((int)s >= 0 && s < MM_ERR_LAST) ? names[s] : "unknown status";
}

void mmb_log(int lvl, const char *file, int line, const char *fmt, ...)
{
    if (lvl < 0 || lvl > 3 || lvl > g_level)
        return;
    const char *base = strrchr(file, '/');
    va_list ap;
    fprintf(stderr, "%c %s:%d: ", "EWID"[lvl], base ? base + 1 : file, line);
    va_start(ap, fmt);
    vfprintf(stderr, fmt, ap);
    va_end(ap);
    fputc('\n', stderr);
}
