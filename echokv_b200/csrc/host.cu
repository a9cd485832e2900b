// Host-side pieces of the C ABI: error text, layout arithmetic, argument checks.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace echokv {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// TieredLayout.__post_init__ / offsets / per_token_bytes (echokv_vllm/tiered_cache.py:85-147).
int describe(const echokv_layout* l, echokv_layout_info* out) {
  if (!l || !out) return set_error(ECHOKV_E_ARGUMENT, "layout/out is null");
  const int64_t h = l->num_kv_heads, d = l->head_size, bs = l->block_size, kg = l->k_group, vg = l->v_group;
  const int mb = l->mem_bits;
  if (h <= 0 || d <= 0 || bs <= 0 || kg <= 0 || vg <= 0)
    return set_error(ECHOKV_E_LAYOUT, "layout fields must be positive");
  if (!(mb == 2 || mb == 4 || mb == 6 || mb == 8))
    return set_error(ECHOKV_E_LAYOUT, "mem_bits must be one of 2/4/6/8, got %d", mb);
  if (bs % 16 != 0) return set_error(ECHOKV_E_LAYOUT, "block_size must be a multiple of 16, got %d", (int)bs);
  if (bs % kg != 0 || bs / kg > 8)
    return set_error(ECHOKV_E_LAYOUT, "block_size %d must be 1-8 multiples of k_group %d", (int)bs, (int)kg);
  if (d % vg != 0 || d % 4 != 0)
    return set_error(ECHOKV_E_LAYOUT, "head_size %d must be divisible by v_group %d and by 4", (int)d, (int)vg);
  const int64_t ng = d / vg, kgpb = bs / kg;
  out->o_v_scale = bs;
  out->o_v_min = out->o_v_scale + bs * h * ng * 2;
  out->o_k_scale = out->o_v_min + bs * h * ng * 2;
  out->o_k_min = out->o_k_scale + kgpb * h * d * 2;
  out->o_data = out->o_k_min + kgpb * h * d * 2;
  out->chunk_bytes = bs * h * d / 2;
  out->chunks_per_page = mb / 2;
  out->page_bytes = out->o_data + out->chunks_per_page * out->chunk_bytes;
  const int64_t raw = 1 + 4 * h * ng + 4 * h * d / kg + (mb / 2) * h * d / 2;
  out->per_token_bytes = (raw + 3) / 4 * 4;
  out->k_groups_per_block = (int32_t)kgpb;
  out->v_groups = (int32_t)ng;
  out->reserved = 0;
  return ECHOKV_OK;
}

int make_layout(const echokv_layout* l, const echokv_pages* p, LayoutDev* L) {
  echokv_layout_info info;
  int rc = describe(l, &info);
  if (rc) return rc;
  if (!p || !p->base) return set_error(ECHOKV_E_ARGUMENT, "pages is null");
  if (p->page_stride_bytes < info.page_bytes)
    return set_error(ECHOKV_E_ARGUMENT, "page stride %lld is smaller than the layout's page (%lld bytes)",
                     (long long)p->page_stride_bytes, (long long)info.page_bytes);
  if (p->page_stride_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(p->base) % 16) != 0)
    return set_error(ECHOKV_E_ARGUMENT, "pages must be 16-byte aligned with a 16-byte aligned row stride");
  if (l->head_size % 16 != 0 || l->v_group % 8 != 0)
    return set_error(ECHOKV_E_UNSUPPORTED, "kernels need head_size %% 16 == 0 and v_group %% 8 == 0 (got %d, %d)",
                     l->head_size, l->v_group);
  L->H = l->num_kv_heads; L->D = l->head_size; L->BS = l->block_size; L->KG = l->k_group; L->VG = l->v_group;
  L->KC = info.chunks_per_page; L->NG = info.v_groups; L->KGPB = info.k_groups_per_block;
  L->o_vs = info.o_v_scale; L->o_vm = info.o_v_min; L->o_ks = info.o_k_scale; L->o_km = info.o_k_min;
  L->o_data = info.o_data; L->CB = info.chunk_bytes; L->PS = p->page_stride_bytes; L->NB = p->num_blocks;
  return ECHOKV_OK;
}

int make_residual(const echokv_residual* r, ResidualDev* R) {
  if (!r || !r->base || !r->block_res || !r->res_group)
    return set_error(ECHOKV_E_ARGUMENT, "residual buffer / block_res / res_group is null");
  if (r->dtype < ECHOKV_DT_F32 || r->dtype > ECHOKV_DT_BF16)
    return set_error(ECHOKV_E_ARGUMENT, "bad residual dtype %d", r->dtype);
  R->base = r->base; R->dtype = r->dtype;
  R->s_slot = r->s_slot; R->s_pos = r->s_pos; R->s_head = r->s_head;
  R->block_res = r->block_res; R->res_group = r->res_group;
  return ECHOKV_OK;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(ECHOKV_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return ECHOKV_OK;
}

}  // namespace echokv

extern "C" {

int echokv_abi_version(void) { return ECHOKV_ABI_VERSION; }

const char* echokv_last_error(void) { return echokv::g_err; }

int echokv_layout_describe(const echokv_layout* layout, echokv_layout_info* out) {
  return echokv::describe(layout, out);
}

}  // extern "C"
