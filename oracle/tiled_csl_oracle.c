/*
 * TEST INFRASTRUCTURE ONLY -- never linked into, imported by or called from the
 * product library.  This file is a plain-C, single-threaded restatement of the
 * host-side algorithms of the HeteroSparse / Flash-LLM SpMM path, written to be
 * read side by side with the reference sources.  Each function names the
 * reference file:line range it follows.  It is the checker the CUDA path and
 * the product's fast encoder are compared against.
 *
 * Parity status: PINNED.  Every encoder in this file is compared word for word
 * with the reference's own compiled encoder (built from the reference sources
 * into oracle/_ref/ by oracle/Makefile) in tests/test_oracle_pin.py, and with
 * committed fixtures under tests/golden/ that were produced by that compiled
 * reference.
 *
 * fp16 values travel as raw uint16_t bit patterns so no CUDA header is needed.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define OR_TILE_M 128 /* csrc/SpMM_API.cu:249  (_TILE_M of the uint32 formats) */
#define OR_TILE_K 64  /* csrc/TilingConfig.h:29 (TILE_K = MMA_K * BLOCK_K_TENSORS) */
#define OR_VEC 4      /* csrc/SpMM_API.cu:250  (VECTOR_SIZE) */
#define OR_BANKS 32

/* Exact fp16 -> fp32 widening (what host __half2float does). */
float oracle_half_to_float(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp  = (h >> 10) & 0x1fu;
    uint32_t man  = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        }
        else { /* subnormal: renormalise */
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while ((man & 0x400u) == 0);
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    }
    else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    }
    else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* Round-to-nearest-even fp32 -> fp16 (what __float2half_rn does). */
uint16_t oracle_float_to_half(float f)
{
    _Float16 h = (_Float16)f;
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
}

/* The encoders' nonzero test: fabs(__half2float(v)) > 0.0f
 * (csrc/SpMM_API.cu:262,285,335).  False for +0, -0 and NaN; true for
 * subnormals and infinities. */
static int enc_nonzero(uint16_t h)
{
    return fabsf(oracle_half_to_float(h)) > 0.0f;
}

/* decompose's nonzero test: __half2float(v) != 0.0f
 * (kernel_benchmark/spmm_decompose.h:26).  True for NaN, false for -0. */
static int dec_nonzero(uint16_t h)
{
    return oracle_half_to_float(h) != 0.0f;
}

/* A growable stack of 32-bit items standing in for std::vector<unsigned>. */
typedef struct {
    uint32_t* v;
    int       n;
    int       cap;
} stack_t;

static void st_push(stack_t* s, uint32_t x)
{
    if (s->n == s->cap) {
        s->cap = s->cap ? 2 * s->cap : 64;
        s->v   = (uint32_t*)realloc(s->v, (size_t)s->cap * sizeof(uint32_t));
    }
    s->v[s->n++] = x;
}

static uint32_t st_pop(stack_t* s)
{
    return s->v[--s->n];
}

/* csrc/SpMM_API.cu:210-221: first index holding the smallest stack. */
static int bank_min(const stack_t* b)
{
    int id = 0, best = b[0].n;
    for (int i = 1; i < OR_BANKS; i++)
        if (b[i].n < best) {
            id   = i;
            best = b[i].n;
        }
    return id;
}

/* csrc/SpMM_API.cu:223-234: first index holding the largest stack. */
static int bank_max(const stack_t* b)
{
    int id = 0, best = b[0].n;
    for (int i = 1; i < OR_BANKS; i++)
        if (b[i].n > best) {
            id   = i;
            best = b[i].n;
        }
    return id;
}

/* Word layout shared by the uint32 formats (csrc/SpMM_API.cu:336-339): the low
 * half-word is the fp16 value, the high half-word the position as a short. */
static uint32_t make_item(uint16_t value, int position)
{
    return (uint32_t)value | ((uint32_t)(uint16_t)(int16_t)position << 16);
}

/* Padding per tile and the total, csrc/SpMM_API.cu:272-294 (same block in every
 * variant).  Returns the padded total; pad[] gets one entry per tile. */
static long count_padding(const uint16_t* A, int M, int K, int* pad)
{
    long total = 0;
    for (int i = 0; i < M / OR_TILE_M; i++)
        for (int j = 0; j < K / OR_TILE_K; j++) {
            const uint16_t* t   = A + (size_t)(i * OR_TILE_M) * K + j * OR_TILE_K;
            int             nnz = 0;
            for (int m = 0; m < OR_TILE_M; m++)
                for (int n = 0; n < OR_TILE_K; n++)
                    if (enc_nonzero(t[(size_t)m * K + n]))
                        nnz++;
            int p                        = (OR_VEC - (nnz % OR_VEC)) % OR_VEC;
            pad[i * (K / OR_TILE_K) + j] = p;
            total += nnz + p;
        }
    return total;
}

/*
 * Tiled-CSL with ahead-of-time bank reordering.
 * Follows InitSparseMatrixA_API, csrc/SpMM_API.cu:241-438, step by step:
 *   scan + bucket by shared-memory bank      :326-349
 *   pad to a multiple of four                 :352-365
 *   tail part drawn from the fullest banks    :384-391
 *   main part drawn from the fullest banks    :394-403
 *   LIFO emission, lane-interleaved           :406-424
 *   offsets in units of four words            :426-435
 * Returns the number of TileOffsets entries (tiles + 2), :437.
 */
int oracle_init_sparse_matrix_a(const uint16_t* A, int M, int K, uint32_t** words_out, int** offsets_out)
{
    if (M % OR_TILE_M || K % OR_TILE_K)
        return -1;
    const int tiles_m = M / OR_TILE_M, tiles_k = K / OR_TILE_K;
    int*      pad   = (int*)malloc((size_t)tiles_m * tiles_k * sizeof(int) + 4);
    long      total = count_padding(A, M, K, pad);
    uint32_t* words = (uint32_t*)malloc((size_t)total * 4 + 16);
    int*      offs  = (int*)malloc(((size_t)tiles_m * tiles_k + 2) * sizeof(int));
    stack_t   bank[OR_BANKS], main_part[OR_BANKS], tail_part[OR_BANKS];
    memset(bank, 0, sizeof bank);
    memset(main_part, 0, sizeof main_part);
    memset(tail_part, 0, sizeof tail_part);

    long      running = 0;
    uint32_t* out     = words;
    for (int i = 0; i < tiles_m; i++)
        for (int j = 0; j < tiles_k; j++) {
            const uint16_t* t = A + (size_t)(i * OR_TILE_M) * K + j * OR_TILE_K;
            int             zero_pos[OR_BANKS];
            int             count = 0;
            for (int b = 0; b < OR_BANKS; b++) {
                bank[b].n = main_part[b].n = tail_part[b].n = 0;
                zero_pos[b]                                  = -1;
            }
            for (int m = 0; m < OR_TILE_M; m++)
                for (int n = 0; n < OR_TILE_K; n++) {
                    uint16_t v   = t[(size_t)m * K + n];
                    int      cp  = n ^ ((m % 8) << 3);    /* :332-333 */
                    int      bk  = (cp / 2) % OR_BANKS;   /* :334 */
                    int      pos = m * OR_TILE_K + cp;    /* :339 */
                    if (enc_nonzero(v)) {
                        st_push(&bank[bk], make_item(v, pos));
                        count++;
                    }
                    else if (zero_pos[bk] == -1) {
                        zero_pos[bk] = pos; /* :345-346 */
                    }
                }
            for (int k = 0; k < pad[i * tiles_k + j]; k++) { /* :352-365 */
                int b = bank_min(bank);
                st_push(&bank[b], make_item(0, zero_pos[b]));
                count++;
            }
            int vectors = count / OR_VEC;
            int repeat  = vectors / 32;
            int rem     = vectors % 32;
            for (int v = 0; v < OR_VEC; v++) /* :384-391 */
                for (int b = 0; b < rem; b++) {
                    int src = bank_max(bank);
                    st_push(&tail_part[b], st_pop(&bank[src]));
                }
            for (int r = 0; r < repeat; r++) /* :394-403 */
                for (int v = 0; v < OR_VEC; v++)
                    for (int b = 0; b < 32; b++) {
                        int src = bank_max(bank);
                        st_push(&main_part[b], st_pop(&bank[src]));
                    }
            for (int r = 0; r < repeat; r++) /* :406-415 */
                for (int v = 0; v < OR_VEC; v++)
                    for (int b = 0; b < 32; b++)
                        out[r * OR_VEC * 32 + b * OR_VEC + v] = st_pop(&main_part[b]);
            out += repeat * OR_VEC * 32;
            for (int v = 0; v < OR_VEC; v++) /* :417-423 */
                for (int b = 0; b < rem; b++)
                    out[b * OR_VEC + v] = st_pop(&tail_part[b]);
            out += OR_VEC * rem;
            running += count;
            offs[i * tiles_k + j + 1] = (int)(running / OR_VEC); /* :427 */
        }
    offs[0]                     = 0;
    offs[tiles_m * tiles_k + 1] = (int)(running / OR_VEC); /* :432-435 */
    for (int b = 0; b < OR_BANKS; b++) {
        free(bank[b].v);
        free(main_part[b].v);
        free(tail_part[b].v);
    }
    free(pad);
    *words_out   = words;
    *offsets_out = offs;
    return tiles_m * tiles_k + 2;
}

/*
 * Tiled-CSL in plain scan order.  Follows InitSparseMatrixA_API_NoReorder,
 * csrc/SpMM_API.cu:441-567: nonzeros in row-major order; the tile's padding
 * words are the first zeros met during the scan and carry that element's own
 * bits (so a -0 or NaN pad keeps its pattern), :534-549.
 */
int oracle_init_sparse_matrix_a_noreorder(const uint16_t* A, int M, int K, uint32_t** words_out, int** offsets_out)
{
    if (M % OR_TILE_M || K % OR_TILE_K)
        return -1;
    const int tiles_m = M / OR_TILE_M, tiles_k = K / OR_TILE_K;
    int*      pad   = (int*)malloc((size_t)tiles_m * tiles_k * sizeof(int) + 4);
    long      total = count_padding(A, M, K, pad);
    uint32_t* words = (uint32_t*)malloc((size_t)total * 4 + 16);
    int*      offs  = (int*)malloc(((size_t)tiles_m * tiles_k + 2) * sizeof(int));
    long      n_out = 0;
    for (int i = 0; i < tiles_m; i++)
        for (int j = 0; j < tiles_k; j++) {
            const uint16_t* t         = A + (size_t)(i * OR_TILE_M) * K + j * OR_TILE_K;
            int             remaining = pad[i * tiles_k + j];
            for (int m = 0; m < OR_TILE_M; m++)
                for (int n = 0; n < OR_TILE_K; n++) {
                    uint16_t v   = t[(size_t)m * K + n];
                    int      pos = m * OR_TILE_K + (n ^ ((m % 8) << 3));
                    if (enc_nonzero(v)) {
                        words[n_out++] = make_item(v, pos);
                    }
                    else if (remaining > 0) {
                        remaining--;
                        words[n_out++] = make_item(v, pos);
                    }
                }
            offs[i * tiles_k + j + 1] = (int)(n_out / OR_VEC);
        }
    offs[0]                     = 0;
    offs[tiles_m * tiles_k + 1] = (int)(n_out / OR_VEC);
    free(pad);
    *words_out   = words;
    *offsets_out = offs;
    return tiles_m * tiles_k + 2;
}

/*
 * Inverse of the uint32 tiled-CSL formats: what the consuming kernel does with
 * each word -- store the value at half-word `position` of a zeroed 128x64 tile
 * (the scatter the reference's dense pipeline was built around,
 * csrc/MMA_PTX.cuh:26-31 undoes the same XOR when it reads the tile back) --
 * followed by un-permuting the columns.  dense must hold M*K half-words.
 * Returns 0, or -1 when an offset or position is out of range.
 */
int oracle_decode_tiled_csl(const uint32_t* words, const int* offsets, int M, int K, uint16_t* dense)
{
    const int tiles_m = M / OR_TILE_M, tiles_k = K / OR_TILE_K;
    memset(dense, 0, (size_t)M * K * 2);
    for (int i = 0; i < tiles_m; i++)
        for (int j = 0; j < tiles_k; j++) {
            int  t  = i * tiles_k + j;
            long w0 = (long)offsets[t] * OR_VEC, w1 = (long)offsets[t + 1] * OR_VEC;
            if (w1 < w0)
                return -1;
            for (long w = w0; w < w1; w++) {
                uint16_t v   = (uint16_t)(words[w] & 0xffffu);
                int      pos = (int)(words[w] >> 16);
                if (pos >= OR_TILE_M * OR_TILE_K)
                    return -1;
                int row = pos / OR_TILE_K;
                int col = (pos % OR_TILE_K) ^ ((row % 8) << 3);
                if ((v & 0x7fffu) != 0) /* padding words carry zero to a zero slot */
                    dense[(size_t)(i * OR_TILE_M + row) * K + j * OR_TILE_K + col] = v;
            }
        }
    return 0;
}

/*
 * Host product in the precision the GPU path promises: fp16 inputs widened
 * exactly, fp32 accumulation with k ascending, one rounding to fp16 at the end.
 * A is dense row-major [M][K], B row-major [K][N], C row-major [M][N] -- the
 * layouts the live kernel uses (csrc/SpMM_Kernel.cuh:372-374, :731-734).  The
 * reference has no host product (its truth is cuBLAS,
 * kernel_benchmark/spmm_test.cu:150-283); this one stands in for it.
 */
void oracle_spmm_f32(const uint16_t* A, const uint16_t* B, uint16_t* C, int M, int N, int K)
{
    float* brow = (float*)malloc((size_t)K * N * sizeof(float));
    for (size_t x = 0; x < (size_t)K * N; x++)
        brow[x] = oracle_half_to_float(B[x]);
    float* acc = (float*)malloc((size_t)N * sizeof(float));
    for (int m = 0; m < M; m++) {
        for (int n = 0; n < N; n++)
            acc[n] = 0.0f;
        for (int k = 0; k < K; k++) {
            uint16_t a = A[(size_t)m * K + k];
            if ((a & 0x7fffu) == 0)
                continue;
            float        af = oracle_half_to_float(a);
            const float* b  = brow + (size_t)k * N;
            for (int n = 0; n < N; n++)
                acc[n] += af * b[n];
        }
        for (int n = 0; n < N; n++)
            C[(size_t)m * N + n] = oracle_float_to_half(acc[n]);
    }
    free(acc);
    free(brow);
}

/* The tolerance oracle: the same product in fp64, no final rounding. */
void oracle_spmm_f64(const uint16_t* A, const uint16_t* B, double* C, int M, int N, int K)
{
    double* brow = (double*)malloc((size_t)K * N * sizeof(double));
    for (size_t x = 0; x < (size_t)K * N; x++)
        brow[x] = (double)oracle_half_to_float(B[x]);
    double* acc = (double*)malloc((size_t)N * sizeof(double));
    for (int m = 0; m < M; m++) {
        for (int n = 0; n < N; n++)
            acc[n] = 0.0;
        for (int k = 0; k < K; k++) {
            uint16_t a = A[(size_t)m * K + k];
            if ((a & 0x7fffu) == 0)
                continue;
            double        af = (double)oracle_half_to_float(a);
            const double* b  = brow + (size_t)k * N;
            for (int n = 0; n < N; n++)
                acc[n] += af * b[n];
        }
        for (int n = 0; n < N; n++)
            C[(size_t)m * N + n] = acc[n];
    }
    free(acc);
    free(brow);
}

/*
 * The reference's CPU SpMM as the harness would run it: decode the tiled-CSL
 * words back to a dense tile, then the fp32-accumulate product above.  Used as
 * the timed CPU baseline (kind "port") and to check the GPU result.
 */
int oracle_spmm_from_csl(const uint32_t* words, const int* offsets, const uint16_t* B, uint16_t* C, int M, int N, int K)
{
    uint16_t* dense = (uint16_t*)malloc((size_t)M * K * 2);
    int       rc    = oracle_decode_tiled_csl(words, offsets, M, K, dense);
    if (rc == 0)
        oracle_spmm_f32(dense, B, C, M, N, K);
    free(dense);
    return rc;
}

/*
 * 2:4 + residual split.  Follows decompose,
 * kernel_benchmark/spmm_decompose.h:12-51: in every aligned group of four
 * consecutive elements the first two nonzeros go to A1, later ones to A2.
 */
void oracle_decompose(const uint16_t* A, uint16_t* A1, uint16_t* A2, int length)
{
    memset(A1, 0, (size_t)length * 2);
    memset(A2, 0, (size_t)length * 2);
    for (int i = 0; i + 3 < length; i += 4) {
        int taken = 0;
        for (int x = 0; x < 4; x++)
            if (dec_nonzero(A[i + x])) {
                if (taken < 2)
                    A1[i + x] = A[i + x];
                else
                    A2[i + x] = A[i + x];
                taken++;
            }
    }
}

/*
 * Variant that sends groups with at most one nonzero wholly to A2.  Follows
 * decompose_v1, kernel_benchmark/spmm_decompose.h:53-142.
 */
void oracle_decompose_v1(const uint16_t* A, uint16_t* A1, uint16_t* A2, int length)
{
    memset(A1, 0, (size_t)length * 2);
    memset(A2, 0, (size_t)length * 2);
    for (int i = 0; i + 3 < length; i += 4) {
        int nnz = 0;
        for (int x = 0; x < 4; x++)
            nnz += dec_nonzero(A[i + x]);
        int taken = 0;
        for (int x = 0; x < 4; x++)
            if (dec_nonzero(A[i + x])) {
                if (nnz > 1 && taken < 2) {
                    A1[i + x] = A[i + x];
                    taken++;
                }
                else {
                    A2[i + x] = A[i + x];
                }
            }
    }
}

/*
 * Seeded synthetic inputs for the CPU-side legs of the benchmark (no counterpart in the reference,
 * whose harness draws from rand(), kernel_benchmark/spmm_test_utils.h:108-162): element i of a
 * stream is fp16(sigma * gaussian), zeroed with probability p_zero, from three counter-based
 * splitmix64 uniforms (Box-Muller).  Written here independently so that the CPU legs need nothing
 * from the product library; tests compare the two generators bit for bit.  Fills the rows x cols
 * block at (row0, col0) of a virtual row-major matrix with ld columns.
 */
static uint64_t synth_mix(uint64_t seed, uint64_t index)
{
    uint64_t z = seed + (index + 1) * 0x9e3779b97f4a7c15ull;
    z          = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z          = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

static double synth_unit(uint64_t x)
{
    return ((double)(x >> 11) + 0.5) * (1.0 / 9007199254740992.0);
}

void oracle_synth_fp16_block(uint16_t* out, long rows, long cols, long ld, long row0, long col0, uint64_t seed, double sigma,
                             double p_zero)
{
    for (long r = 0; r < rows; r++)
        for (long c = 0; c < cols; c++) {
            const uint64_t base = (uint64_t)((row0 + r) * ld + col0 + c) * 3u;
            uint16_t       bits = 0;
            if (!(synth_unit(synth_mix(seed, base + 2)) < p_zero)) {
                const double u1 = synth_unit(synth_mix(seed, base));
                const double u2 = synth_unit(synth_mix(seed, base + 1));
                const double g  = sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2);
                bits            = oracle_float_to_half((float)(sigma * g));
            }
            out[r * cols + c] = bits;
        }
}
