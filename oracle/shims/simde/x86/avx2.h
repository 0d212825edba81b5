// Test infrastructure (oracle build only): maps the simde_* spellings the
// reference CPU backend uses onto the native x86 intrinsics of <immintrin.h>.
// On an AVX2/FMA/F16C host simde lowers each of these names to exactly that
// native instruction, so aliasing them changes no arithmetic.
#pragma once
#include <immintrin.h>

typedef __m128  simde__m128;
typedef __m128i simde__m128i;
typedef __m256  simde__m256;
typedef __m256i simde__m256i;

#define SIMDE_MM_ROUND_NEAREST          (_MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC)
#define SIMDE_MM_FROUND_TO_NEAREST_INT  _MM_FROUND_TO_NEAREST_INT
#define SIMDE_MM_SHUFFLE(z, y, x, w)    _MM_SHUFFLE(z, y, x, w)

// 256-bit float
#define simde_mm256_setzero_ps          _mm256_setzero_ps
#define simde_mm256_set1_ps             _mm256_set1_ps
#define simde_mm256_loadu_ps            _mm256_loadu_ps
#define simde_mm256_storeu_ps           _mm256_storeu_ps
#define simde_mm256_add_ps              _mm256_add_ps
#define simde_mm256_sub_ps              _mm256_sub_ps
#define simde_mm256_mul_ps              _mm256_mul_ps
#define simde_mm256_div_ps              _mm256_div_ps
#define simde_mm256_max_ps              _mm256_max_ps
#define simde_mm256_andnot_ps           _mm256_andnot_ps
#define simde_mm256_fmadd_ps            _mm256_fmadd_ps
#define simde_mm256_round_ps(a, mode)   _mm256_round_ps((a), (mode))
#define simde_mm256_cvtps_epi32         _mm256_cvtps_epi32
#define simde_mm256_cvtepi32_ps         _mm256_cvtepi32_ps
#define simde_mm256_castps256_ps128     _mm256_castps256_ps128
#define simde_mm256_extractf128_ps(a, i) _mm256_extractf128_ps((a), (i))
#define simde_mm256_cvtph_ps            _mm256_cvtph_ps
#define simde_mm256_cvtps_ph(a, mode)   _mm256_cvtps_ph((a), (mode))

// 256-bit integer
#define simde_mm256_set1_epi16          _mm256_set1_epi16
#define simde_mm256_setr_epi32          _mm256_setr_epi32
#define simde_mm256_set_m128i           _mm256_set_m128i
#define simde_mm256_add_epi32           _mm256_add_epi32
#define simde_mm256_sign_epi8           _mm256_sign_epi8
#define simde_mm256_maddubs_epi16       _mm256_maddubs_epi16
#define simde_mm256_madd_epi16          _mm256_madd_epi16
#define simde_mm256_packs_epi32         _mm256_packs_epi32
#define simde_mm256_packs_epi16         _mm256_packs_epi16
#define simde_mm256_permutevar8x32_epi32 _mm256_permutevar8x32_epi32
#define simde_mm256_castsi256_si128     _mm256_castsi256_si128
#define simde_mm256_extractf128_si256(a, i) _mm256_extractf128_si256((a), (i))

static inline __m256i simde_mm256_loadu_si256(const void *p) { return _mm256_loadu_si256(static_cast<const __m256i *>(p)); }
static inline void    simde_mm256_storeu_si256(void *p, __m256i v) { _mm256_storeu_si256(static_cast<__m256i *>(p), v); }

// 128-bit float
#define simde_mm_add_ps                 _mm_add_ps
#define simde_mm_add_ss                 _mm_add_ss
#define simde_mm_max_ps                 _mm_max_ps
#define simde_mm_max_ss                 _mm_max_ss
#define simde_mm_hadd_ps                _mm_hadd_ps
#define simde_mm_movehl_ps              _mm_movehl_ps
#define simde_mm_movehdup_ps            _mm_movehdup_ps
#define simde_mm_cvtss_f32              _mm_cvtss_f32

// 128-bit integer
#define simde_mm_set1_epi8              _mm_set1_epi8
#define simde_mm_set1_epi16             _mm_set1_epi16
#define simde_mm_and_si128              _mm_and_si128
#define simde_mm_sub_epi8               _mm_sub_epi8
#define simde_mm_add_epi32              _mm_add_epi32
#define simde_mm_sign_epi8              _mm_sign_epi8
#define simde_mm_maddubs_epi16          _mm_maddubs_epi16
#define simde_mm_madd_epi16             _mm_madd_epi16
#define simde_mm_srli_epi64(a, i)       _mm_srli_epi64((a), (i))
#define simde_mm_unpackhi_epi64         _mm_unpackhi_epi64
#define simde_mm_shuffle_epi32(a, i)    _mm_shuffle_epi32((a), (i))
#define simde_mm_cvtsi128_si32          _mm_cvtsi128_si32

static inline __m128i simde_mm_loadu_si128(const void *p) { return _mm_loadu_si128(static_cast<const __m128i *>(p)); }
static inline void    simde_mm_storeu_si128(void *p, __m128i v) { _mm_storeu_si128(static_cast<__m128i *>(p), v); }
