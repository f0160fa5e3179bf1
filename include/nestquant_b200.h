/*
 * nestquant_b200 C ABI: the NestQuant quantized routed-expert MoE layer on NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device/host pointers and sizes, enqueues its work on `stream`
 * (a cudaStream_t passed as void*; NULL = the legacy default stream), never synchronises and
 * returns 0 or a negative NQ_ERR_* code.  nq_last_error() gives the message of the calling thread's last failure.
 * Unless a function says otherwise it allocates nothing: all memory is caller-owned.
 *
 * Each declaration names the interface of the reference implementation (jarrelscy/nestquant) that it
 * replaces, as file:line of that project.  The reference binds these through a torch C++ extension
 * (sm120/nqmoe.cu:1294-1295); a ctypes binding with the same Python-visible names ships in nestquant_b200/ext.py.
 *
 * Device table: int64 [E][20] per layer, one row per expert (sm120/nqmoe.cu:26-45, sm120/moe.py:216-229):
 *   [0] level (0 = not resident here, 2, 4)   [1..4] gate|up: base, p4, d4, flags (0 = dense)   [5..8] down: same
 *   [9] fp16 scales [H su_g | I sv_g | I sv_u | I su_d | H sv_o | H su_u]   [10],[11] residual window codes
 *   [12],[13] ring-sign planes (0 = none)   [14] low-rank plane, [15] its level-4 part, [16] r_gu, [17] r_dn
 *   [18] width of the down-input rotation (0 or 128, or 512)   [19] base window codes (must be 0)
 */
#ifndef NESTQUANT_B200_H
#define NESTQUANT_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NQ_TABLE_WIDTH 20
#define NQ_MAX_TOKENS 32          /* tokens per decode-path call */
#define NQ_MAX_PICKS 256          /* tokens * topk per decode-path call */

enum {
    NQ_OK = 0,
    NQ_ERR_ARG = -1,              /* bad shape, size, alignment or configuration */
    NQ_ERR_CUDA = -2,             /* a CUDA runtime call or launch failed */
    NQ_ERR_UNSUPPORTED = -3       /* valid in the format but not built into this library */
};

const char* nq_last_error(void);
/* library build info: compute capability it was compiled for (100), as a sanity check for loaders */
int nq_build_arch(void);

/* Residual window codes compiled in, bit c = code c: out[0] gate|up, out[1] down.
 * Replaces rk_codes() (sm120/nqmoe.cu:938-940). */
int nq_rk_codes(int64_t out[2]);
/* Base window codes compiled in (bit 0 only: the 128-bit ring base).  Replaces the optional bk_codes()
 * that sm120/moe.py:247-249 probes for. */
int nq_bk_codes(int64_t out[2]);

/* Bytes of a residual plane of `nrec` lane records of window code `code` (sm120/moe.py:27-30), or 0 for a bad code. */
size_t nq_plane_bytes(size_t nrec, int code);

/* Dense decode of `n_experts` experts to fp16 matrices, level and pointers read from the live table rows:
 * Wgu [n][2I][H], Wdn [n][H][I] (either may be NULL to skip that projection); experts = int32 expert ids (device).
 * Level-0 experts decode to zeros.  Replaces pf_decode() (sm120/nqmoe.cu:1013-1080,1247-1257) and, with one expert,
 * the NQ_WDUMP debug hook set_wdump() (sm120/nqmoe.cu:246-248,852-853) used for the bit-exactness checks. */
int nq_pf_decode(const int64_t* table, const int32_t* experts, int n_experts, void* Wgu, void* Wdn,
                 int H, int I, int nm_gu, int nm_dn, int force_level, void* stream);

/* Graph-safe table switch: table[e] = stage[e] wherever seq[e] != applied[e], then applied[e] = seq[e]
 * (also mirrored to applied_host when it is not NULL; host-mapped memory).  Replaces mailbox()
 * (sm120/nqmoe.cu:908-929). */
int nq_mailbox(int64_t* table, const int64_t* stage, const int32_t* seq, int32_t* applied, int32_t* applied_host,
               int E, void* stream);

#ifdef __cplusplus
}
#endif
#endif
