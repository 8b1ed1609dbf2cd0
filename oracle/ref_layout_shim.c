/* TEST INFRASTRUCTURE — NOT PRODUCT CODE.
 *
 * 64-bit-clean shim around the reference project's own layout leaves.  The
 * leaves (qcom_hexagon_backend/bin/runtime/hmx/src/HMXLayout.c) take 32-bit
 * addresses, exactly as on the device, so this shim maps three scratch buffers
 * below 2 GiB, copies the caller's data in, calls the leaf, and copies the
 * result out.  The reference source is compiled where it lies (the Makefile
 * puts the reference tree on the include path); nothing of it is copied here.
 * Build only through oracle/Makefile (target "ref"), output in oracle/_ref/.
 */
#define _GNU_SOURCE
#include <stdint.h>
#include <string.h>
#include <sys/mman.h>

#include "HMXLayout.c" /* found through -I<reference>/qcom_hexagon_backend/bin/runtime/hmx/src */

#if !defined(HMX_HOST_EMU_HEXAGON_TYPES_STUB)
#error "the reference's host stub <hexagon_types.h> must be first on the include path"
#endif

#define REF_BUF_BYTES (24u << 20)
#define REF_GUARD 4096u

static unsigned char *buf_s, *buf_d, *buf_r;

static unsigned char *map_low(size_t n) {
  void *p = mmap(NULL, n, PROT_READ | PROT_WRITE,
                 MAP_PRIVATE | MAP_ANONYMOUS | MAP_32BIT, -1, 0);
  if (p == MAP_FAILED) return NULL;
  if ((uintptr_t)p + n >= (1ull << 31)) return NULL;
  return (unsigned char *)p;
}

int ref_layout_init(void) {
  if (buf_s) return 0;
  buf_s = map_low(REF_BUF_BYTES);
  buf_d = map_low(REF_BUF_BYTES);
  buf_r = map_low(REF_BUF_BYTES);
  return (buf_s && buf_d && buf_r) ? 0 : -1;
}

static unsigned lo32(const void *p) { return (unsigned)(uintptr_t)p; }
static size_t cap(void) { return REF_BUF_BYTES - 2u * REF_GUARD; }

/* [K, N] row-major fp16 -> weight tile image [Nt, Kt] of 2 KiB tiles. */
int ref_pack_weight_f16(const uint16_t *src, uint16_t *dst, unsigned K,
                        unsigned N, unsigned stride) {
  unsigned Kt = (K + 31u) / 32u, Nt = (N + 31u) / 32u;
  size_t sb = (size_t)K * stride * 2u + 256u, db = (size_t)Kt * Nt * 2048u;
  if (ref_layout_init() || sb > cap() || db > cap()) return -1;
  unsigned char *s = buf_s + REF_GUARD, *d = buf_d + REF_GUARD;
  memset(s, 0, sb);
  memcpy(s, src, (size_t)((K - 1) * (size_t)stride + N) * 2u);
  for (unsigned nt = 0; nt < Nt; ++nt)
    hmx_pack_weight_f16_bulk(lo32(d + (size_t)nt * Kt * 2048u), lo32(s), K, N,
                             stride, 0, nt, Kt);
  memcpy(dst, d, db);
  return 0;
}

/* [K, N] row-major fp32 -> fp16 weight tile image (conversion folded in). */
int ref_pack_weight_f32(const float *src, uint16_t *dst, unsigned K, unsigned N,
                        unsigned stride) {
  unsigned Kt = (K + 31u) / 32u, Nt = (N + 31u) / 32u;
  size_t sb = (size_t)K * stride * 4u + 256u, db = (size_t)Kt * Nt * 2048u;
  if (ref_layout_init() || sb > cap() || db > cap()) return -1;
  unsigned char *s = buf_s + REF_GUARD, *d = buf_d + REF_GUARD;
  memset(s, 0, sb);
  memcpy(s, src, (size_t)((K - 1) * (size_t)stride + N) * 4u);
  for (unsigned nt = 0; nt < Nt; ++nt)
    hmx_pack_weight_f32_bulk(lo32(d + (size_t)nt * Kt * 2048u), lo32(s), K, N,
                             stride, 0, nt, Kt);
  memcpy(dst, d, db);
  return 0;
}

/* [rows, cols] row-major fp16 -> activation tile grid [Mt, Kt]. */
int ref_pack_act_f16(const uint16_t *src, uint16_t *dst, unsigned rows,
                     unsigned cols, unsigned stride) {
  unsigned Mt = (rows + 31u) / 32u, Kt = (cols + 31u) / 32u;
  size_t sb = (size_t)rows * stride * 2u + 256u, db = (size_t)Mt * Kt * 2048u;
  if (ref_layout_init() || sb > cap() || db > cap()) return -1;
  unsigned char *s = buf_s + REF_GUARD, *d = buf_d + REF_GUARD;
  memset(s, 0, sb);
  memcpy(s, src, (size_t)((rows - 1) * (size_t)stride + cols) * 2u);
  for (unsigned mt = 0; mt < Mt; ++mt)
    hmx_pack_act_f16_bulk(lo32(d + (size_t)mt * Kt * 2048u), lo32(s), rows, cols,
                          stride, mt, 0, Kt);
  memcpy(dst, d, db);
  return 0;
}

/* tile grid [Mt, Nt] -> row-major fp16 [rows, cols] with row stride `stride`. */
int ref_unpack_acc_f16(const uint16_t *tiles, uint16_t *dst, unsigned rows,
                       unsigned cols, unsigned stride) {
  unsigned Mt = (rows + 31u) / 32u, Nt = (cols + 31u) / 32u;
  size_t sb = (size_t)Mt * Nt * 2048u, db = (size_t)rows * stride * 2u;
  if (ref_layout_init() || sb > cap() || db > cap()) return -1;
  unsigned char *s = buf_s + REF_GUARD, *d = buf_d + REF_GUARD;
  memcpy(s, tiles, sb);
  memcpy(d, dst, db);
  for (unsigned mt = 0; mt < Mt; ++mt)
    hmx_unpack_acc_f16_bulk(lo32(d), lo32(s + (size_t)mt * Nt * 2048u), rows,
                            cols, stride, mt, 16);
  memcpy(dst, d, db);
  return 0;
}

/* tile grid -> row-major fp32, optional fp32 residual added after widening. */
int ref_unpack_acc_f32(const uint16_t *tiles, float *dst, const float *res,
                       unsigned rows, unsigned cols, unsigned stride) {
  unsigned Mt = (rows + 31u) / 32u, Nt = (cols + 31u) / 32u;
  size_t sb = (size_t)Mt * Nt * 2048u, db = (size_t)rows * stride * 4u;
  if (ref_layout_init() || sb > cap() || db > cap()) return -1;
  unsigned char *s = buf_s + REF_GUARD, *d = buf_d + REF_GUARD,
                *r = buf_r + REF_GUARD;
  memcpy(s, tiles, sb);
  memcpy(d, dst, db);
  if (res) memcpy(r, res, db);
  for (unsigned mt = 0; mt < Mt; ++mt)
    hmx_unpack_acc_f32_bulk(lo32(d), res ? lo32(r) : 0u, res ? 1u : 0u,
                            lo32(s + (size_t)mt * Nt * 2048u), rows, cols,
                            stride, stride, mt, 16);
  memcpy(dst, d, db);
  return 0;
}
