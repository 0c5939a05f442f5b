/*
 * cpu_baseline.c -- the CPU arm timed beside the GPU numbers.
 *
 * TEST / BENCHMARK INFRASTRUCTURE ONLY; never linked into the product.
 *
 * The reference's own CPU path for the AEAD is Go assembly inside
 * golang.org/x/crypto (go.mod:7), which cannot be built here (no Go toolchain,
 * module source not in the tree).  Its stand-in is OpenSSL's
 * EVP_chacha20_poly1305 (hand-written AVX2/AVX-512 assembly, the same class of
 * code), driven the way wireguard-go drives x/crypto: one worker thread per core,
 * each sealing or opening whole packets in place with nonce = 0^32 | le64(counter)
 * and the 16-byte transport header in front.  Output is byte-identical to the
 * scalar checker in bnk_oracle.c (tests compare them).
 */
#define _GNU_SOURCE
#include <openssl/evp.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <unistd.h>

#include "bnk_oracle.h"

typedef struct {
    const uint8_t *keys;
    const uint32_t *remote_index;
    uint8_t *ring;
    const uint32_t *off, *len, *slot;
    uint64_t *counter;
    uint8_t *status;
    uint32_t *out_len;
    size_t begin, end, mtu;
    int open;
} job_t;

static double now_s(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

static void st32(uint8_t *p, uint32_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); p[2] = (uint8_t)(v >> 16); p[3] = (uint8_t)(v >> 24); }
static void st64(uint8_t *p, uint64_t v) { st32(p, (uint32_t)v); st32(p + 4, (uint32_t)(v >> 32)); }
static uint32_t ld32(const uint8_t *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }
static uint64_t ld64(const uint8_t *p) { return (uint64_t)ld32(p) | ((uint64_t)ld32(p + 4) << 32); }

static void *worker(void *arg) {
    job_t *j = (job_t *)arg;
    EVP_CIPHER_CTX *c = EVP_CIPHER_CTX_new();
    uint8_t nonce[12] = {0};
    int outl = 0;
    if (j->open) {
        EVP_DecryptInit_ex(c, EVP_chacha20_poly1305(), NULL, NULL, NULL);
        EVP_CIPHER_CTX_ctrl(c, EVP_CTRL_AEAD_SET_IVLEN, 12, NULL);
        for (size_t i = j->begin; i < j->end; i++) {
            uint8_t *p = j->ring + j->off[i];
            uint32_t m = j->len[i];
            if (m < 32 || ld32(p) != 4) {
                j->status[i] = BNKO_MALFORMED;
                j->out_len[i] = 0;
                j->counter[i] = 0;
                continue;
            }
            uint64_t ctr = ld64(p + 8);
            j->counter[i] = ctr;
            st64(nonce + 4, ctr);
            uint32_t body = m - 32;
            EVP_DecryptInit_ex(c, NULL, NULL, j->keys + 32u * j->slot[i], nonce);
            EVP_CIPHER_CTX_ctrl(c, EVP_CTRL_AEAD_SET_TAG, 16, p + 16 + body);
            int ok = EVP_DecryptUpdate(c, p + 16, &outl, p + 16, (int)body) == 1;
            ok = ok && EVP_DecryptFinal_ex(c, p + 16 + body, &outl) == 1;
            if (ok) {
                j->status[i] = body ? BNKO_OK : BNKO_KEEPALIVE;
                j->out_len[i] = body;
            } else {
                memset(p + 16, 0, body);
                j->status[i] = BNKO_AUTH_FAIL;
                j->out_len[i] = 0;
            }
        }
    } else {
        EVP_EncryptInit_ex(c, EVP_chacha20_poly1305(), NULL, NULL, NULL);
        EVP_CIPHER_CTX_ctrl(c, EVP_CTRL_AEAD_SET_IVLEN, 12, NULL);
        for (size_t i = j->begin; i < j->end; i++) {
            uint8_t *p = j->ring + j->off[i];
            uint64_t ctr = j->counter[i];
            if (ctr >= BNKO_REJECT_AFTER_MESSAGES) {
                j->status[i] = BNKO_COUNTER_EXHAUSTED;
                j->out_len[i] = 0;
                continue;
            }
            size_t len = j->len[i], body = bnko_wg_padded_len(len, j->mtu);
            memset(p + 16 + len, 0, body - len);
            st32(p, 4);
            st32(p + 4, j->remote_index[j->slot[i]]);
            st64(p + 8, ctr);
            st64(nonce + 4, ctr);
            EVP_EncryptInit_ex(c, NULL, NULL, j->keys + 32u * j->slot[i], nonce);
            EVP_EncryptUpdate(c, p + 16, &outl, p + 16, (int)body);
            EVP_EncryptFinal_ex(c, p + 16 + body, &outl);
            EVP_CIPHER_CTX_ctrl(c, EVP_CTRL_AEAD_GET_TAG, 16, p + 16 + body);
            j->status[i] = BNKO_OK;
            j->out_len[i] = (uint32_t)(32 + body);
        }
    }
    EVP_CIPHER_CTX_free(c);
    return NULL;
}

int bnkb_host_cores(void) { return (int)sysconf(_SC_NPROCESSORS_ONLN); }

/* Seals (open=0) or opens (open=1) packets [0, n) in place with `threads` workers, each taking a
 * contiguous share.  Returns the wall-clock seconds the workers took. */
double bnkb_aead_batch(int open, int threads, const uint8_t *keys, const uint32_t *remote_index, size_t mtu,
                       uint8_t *ring, const uint32_t *off, const uint32_t *len, const uint32_t *slot,
                       uint64_t *counter, uint8_t *status, uint32_t *out_len, size_t n) {
    if (threads < 1) threads = 1;
    if ((size_t)threads > n && n) threads = (int)n;
    pthread_t *tid = (pthread_t *)calloc((size_t)threads, sizeof *tid);
    job_t *jobs = (job_t *)calloc((size_t)threads, sizeof *jobs);
    double t0 = now_s();
    for (int t = 0; t < threads; t++) {
        job_t *j = &jobs[t];
        j->keys = keys; j->remote_index = remote_index; j->ring = ring; j->off = off; j->len = len; j->slot = slot;
        j->counter = counter; j->status = status; j->out_len = out_len; j->mtu = mtu; j->open = open;
        j->begin = n * (size_t)t / (size_t)threads;
        j->end = n * (size_t)(t + 1) / (size_t)threads;
        pthread_create(&tid[t], NULL, worker, j);
    }
    for (int t = 0; t < threads; t++) pthread_join(tid[t], NULL);
    double dt = now_s() - t0;
    free(tid);
    free(jobs);
    return dt;
}
