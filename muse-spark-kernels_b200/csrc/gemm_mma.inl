// Role body of moe_gemm_kernel (included inside the kernel): MMA issuer, warp 1.
// One A slot (128 K, 64 TMEM columns per tile) is consumed by eight K=16 MMAs per tile and
// handed back with a tcgen05.commit, so several dequant -> MMA -> release hand-offs are in
// flight at once. The accumulators of consecutive units alternate between NDBUF buffers.
    constexpr uint32_t idesc = idesc_f16(FMT_F16, FMT_F16, 128, N);
    uint32_t it = 0, unit_i = 0, sc = 0;
    uint32_t as = 0, apar = 0;  // A ring position and its phase parity
#ifdef MSK_EXP_MMA_CLOCKS
    long long ck_afull = 0, ck_issue = 0, ck_bfull = 0, ck_dempty = 0, ck0 = 0;
    const long long ck_start = clock64();
#define CK_BEGIN() ck0 = clock64()
#define CK_END(acc) acc += clock64() - ck0
#else
#define CK_BEGIN()
#define CK_END(acc)
#endif
    bool ok = true;
    for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++unit_i) {
      const UnitInfo ui = decode_unit(u, tile_start, p, N);
      const int ks0 = ui.split * per_split, ks1 = min(nst_total, ks0 + per_split);
      const uint32_t db = unit_i % NDBUF, duse = unit_i / NDBUF;
      CK_BEGIN();
      if (!mbar_wait(&ctl.d_empty[db], (duse & 1u) ^ 1u, abortw)) { ok = false; break; }
      CK_END(ck_dempty);
      tc_fence_after();
      const uint32_t d_tmem = tmem + db * (2 * N);
      for (int ks = ks0; ks < ks1 && ok; ++ks, ++it) {
        const uint32_t slot = it % NST, par = (it / NST) & 1u;
        CK_BEGIN();
        if (!mbar_wait(&ctl.b_full[slot], par, abortw)) { ok = false; break; }
        CK_END(ck_bfull);
        const uint32_t b_addr = smem_u32(ring + slot * C::STAGE_BYTES + 2 * TILE_BYTES);
#pragma unroll
        for (int sl = 0; sl < 2; ++sl, ++sc) {
          CK_BEGIN();
          if (!mbar_wait(&ctl.a_full[0][as], apar, abortw) || !mbar_wait(&ctl.a_full[1][as], apar, abortw)) {
            ok = false;
            break;
          }
          CK_END(ck_afull);
          CK_BEGIN();
          tc_fence_after();
          if (elect_one()) {  // warp-uniform control flow keeps addresses and descriptors in uniform registers
            if (sc == 0) MSK_TR(TR_FIRST_MMA);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const int k16 = sl * 8 + kk;
              const uint64_t bdesc = C::TMA_B ? smem_desc_kmajor_sw128(b_addr + (k16 >> 2) * (N * 128) + (k16 & 3) * 32)
                                              : smem_desc_kmajor_noswz(b_addr + k16 * 256, B_LBO, B_SBO);
              const uint32_t acc = (ks > ks0 || k16 > 0) ? 1u : 0u;
              mma_ts(d_tmem, tmem + C::A_BASE + as * C::SLOT_COLS + kk * 8, bdesc, idesc, acc);
              mma_ts(d_tmem + N, tmem + C::A_BASE + C::A_GROUP_COLS + as * C::SLOT_COLS + kk * 8, bdesc, idesc, acc);
            }
            tc_commit(&ctl.a_empty[as]);
          }
          __syncwarp();
          CK_END(ck_issue);
          if (++as == NSLOT) { as = 0; apar ^= 1u; }
        }
        if (!ok) break;
        if (elect_one()) tc_commit(&ctl.b_empty[slot]);
        __syncwarp();
      }
      if (ok && elect_one()) tc_commit(&ctl.d_full[db]);
      __syncwarp();
    }
#ifdef MSK_EXP_MMA_CLOCKS
    if (lane == 0 && p.trace != nullptr) {
      p.trace[blockIdx.x * 16 + 10] = ck_afull; p.trace[blockIdx.x * 16 + 11] = ck_issue; p.trace[blockIdx.x * 16 + 12] = ck_bfull;
      p.trace[blockIdx.x * 16 + 13] = ck_dempty; p.trace[blockIdx.x * 16 + 14] = clock64() - ck_start; p.trace[blockIdx.x * 16 + 15] = it;
    }
#endif
