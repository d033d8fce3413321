/*
 * Stand-in for core.c when this library's objects are linked into the mimfer
 * tree: mimfer's own mm_status_str and mm_log (src/core/mimfer.c:16-60) are
 * kept, and the library's log sink forwards to them.  Link this file INSTEAD
 * of core.c.
 */
#include <stdarg.h>
#include <stdio.h>

void mm_log(int lvl, const char *file, int line, const char *fmt, ...);   /* include/mimfer/mimfer.h:84 */

void mmb_log(int lvl, const char *file, int line, const char *fmt, ...)
{
    char text[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(text, sizeof text, fmt, ap);
    va_end(ap);
    mm_log(lvl, file, line, "%s", text);      /* same level numbering: 0 error .. 3 debug */
}

/* the library's own verbosity knob has nothing to set here: mimfer's g_mm_log_level rules */
void mm_log_set_level(int level) { (void)level; }
