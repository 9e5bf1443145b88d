/* TEST INFRASTRUCTURE — CPU oracle: the data-directory tensor source shared by the model files:
 * manifest.txt ("data_start N", then "name type offset nelems" per tensor) over an mmap'd GGUF
 * blob (src/bin/engine_gpt2.rs:1279-1284, src/bin/engine_qwen2.rs:519-526). */
#ifndef ORACLE_SRC_H
#define ORACLE_SRC_H
#define _GNU_SOURCE
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <fcntl.h>
#include <unistd.h>
#include <sys/mman.h>
#include <sys/stat.h>

typedef struct {
    int synth;
    uint64_t seed;
    uint8_t *blob; size_t blob_len;
    char **names; uint32_t *types; size_t *offs; size_t *nel; int nt;
} orc_source;

static inline void orc_die(const char *msg, const char *arg) { fprintf(stderr, "oracle: %s %s\n", msg, arg ? arg : ""); abort(); }

static inline void orc_source_open(orc_source *s, const char *dir, const char *blobp) {
    char path[4096], key[128];
    memset(s, 0, sizeof *s);
    int fd = open(blobp, O_RDONLY);
    if (fd < 0) orc_die("cannot open", blobp);
    struct stat st; fstat(fd, &st);
    s->blob_len = st.st_size;
    s->blob = mmap(NULL, s->blob_len, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    snprintf(path, sizeof path, "%s/manifest.txt", dir);
    FILE *f = fopen(path, "r");
    if (!f) orc_die("cannot open", path);
    size_t data_start = 0;
    if (fscanf(f, "%127s %zu", key, &data_start) != 2) orc_die("bad manifest", path);
    int cap = 1024;
    s->names = malloc(sizeof(char *) * cap); s->types = malloc(4 * cap); s->offs = malloc(sizeof(size_t) * cap); s->nel = malloc(sizeof(size_t) * cap);
    char nm[256]; unsigned ty; size_t off, nel;
    while (fscanf(f, "%255s %u %zu %zu", nm, &ty, &off, &nel) == 4) {
        if (s->nt == cap) { cap *= 2; s->names = realloc(s->names, sizeof(char *) * cap); s->types = realloc(s->types, 4 * cap); s->offs = realloc(s->offs, sizeof(size_t) * cap); s->nel = realloc(s->nel, sizeof(size_t) * cap); }
        s->names[s->nt] = strdup(nm); s->types[s->nt] = ty; s->offs[s->nt] = data_start + off; s->nel[s->nt] = nel; s->nt++;
    }
    fclose(f);
}

static inline void orc_source_close(orc_source *s) {
    if (s->blob) munmap(s->blob, s->blob_len);
    for (int i = 0; i < s->nt; i++) free(s->names[i]);
    free(s->names); free(s->types); free(s->offs); free(s->nel);
}

/* tensor by name; *type and *nel receive its manifest entries */
static inline const uint8_t *orc_source_find(const orc_source *s, const char *name, uint32_t *type, size_t *nel) {
    for (int i = 0; i < s->nt; i++)
        if (!strcmp(s->names[i], name)) { *type = s->types[i]; *nel = s->nel[i]; return s->blob + s->offs[i]; }
    orc_die("missing tensor", name);
    return NULL;
}

/* "key value" lines of config.txt; returns 1 and fills val when the key exists */
static inline int orc_config_get(const char *dir, const char *want, char val[128]) {
    char path[4096], key[128], line[512];
    snprintf(path, sizeof path, "%s/config.txt", dir);
    FILE *f = fopen(path, "r");
    if (!f) orc_die("cannot open", path);
    int found = 0;
    while (fgets(line, sizeof line, f))
        if (sscanf(line, "%127s %127s", key, val) == 2 && !strcmp(key, want)) { found = 1; break; }
    fclose(f);
    return found;
}
#endif
