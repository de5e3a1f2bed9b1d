// Role body of moe_gemm_kernel (included inside the kernel): MMA issuers, warps 1 and 3, one per
// tile of the pair (a single issuing warp, sharing its scheduler with four dequant warps, took
// ~29 cycles per MMA and became the limiter of the narrow-tile main loop).
// One A slot (128 K, 64 TMEM columns per tile) is consumed by eight K=16 MMAs per tile and
// handed back with a tcgen05.commit, so several dequant -> MMA -> release hand-offs are in
// flight at once. The accumulators of consecutive pieces alternate between NDBUF buffers.
    constexpr uint32_t idesc = idesc_f16(FMT_F16, FMT_F16, 128, N);
    const int mg = warp == 1 ? 0 : 1;  // warp 1 issues for tile 0, warp 3 for tile 1
    uint32_t it = 0, unit_i = 0, sc = 0;
    uint32_t as = 0, apar = 0;  // A ring position and its phase parity
    int tri = 0;
    (void)tri;
    bool ok = true;
    MSK_PHASES {
      MSK_PHASE_SETUP;
      for (; ok && pieces.next(base, ks0, ks1); ++unit_i) {
        const UnitInfo ui = decode_unit(base, tile_start, pp.n_pairs, p.nloc, N);
        const uint32_t db = unit_i % NDBUF, duse = unit_i / NDBUF;
        if (!MSK_WAIT(&ctl.d_empty[db], (duse & 1u) ^ 1u, abortw)) { ok = false; break; }
        tc_fence_after();
        if (mg == 0 && lane == 0) MSK_TRD(1, tri, 3);
        const uint32_t d_tmem = tmem + db * (2 * N) + mg * N;
        // a ragged last token tile of an expert only pays for the columns it has (MMA N in steps of 16):
        // at N = 128 an MMA costs 64 cycles, at N = 16 nine
        const uint32_t idesc_u = N >= 64 ? idesc_f16(FMT_F16, FMT_F16, 128, static_cast<uint32_t>((ui.rows + 15) & ~15)) : idesc;
        const uint32_t a_base = tmem + C::A_BASE + mg * C::A_GROUP_COLS;
        for (int ks = ks0; ks < ks1 && ok; ++ks, ++it) {
          const uint32_t slot = it % NST, par = (it / NST) & 1u;
#ifdef MSK_TRACE_DETAIL
          if (mg == 0 && lane == 0 && !mbar_test(&ctl.b_full[slot], par)) MSK_TRD(1, tri, 4);   // B tile not there yet
#endif
          if (!MSK_WAIT(&ctl.b_full[slot], par, abortw)) { ok = false; break; }
          if (mg == 0 && lane == 0) MSK_TRD(1, tri, 1);
          const uint32_t b_addr = smem_u32(ring + slot * C::STAGE_BYTES + 2 * TILE_BYTES);
#pragma unroll
          for (int sl = 0; sl < 2; ++sl, ++sc) {
#ifdef MSK_TRACE_DETAIL
            if (mg == 0 && lane == 0 && !mbar_test(&ctl.a_full[mg][as], apar)) MSK_TRD(1, tri, 5);   // A slot not there yet
#endif
            if (!MSK_WAIT(&ctl.a_full[mg][as], apar, abortw)) { ok = false; break; }
            if (mg == 0 && lane == 0) MSK_TRD(1, tri, 6);
            tc_fence_after();
            if (elect_one()) {  // warp-uniform control flow keeps addresses and descriptors in uniform registers
              if (sc == 0 && mg == 0) MSK_TR(TR_FIRST_MMA);
#pragma unroll
              for (int kk = 0; kk < 8; ++kk) {
                const int k16 = sl * 8 + kk;
                const uint64_t bdesc = TMA_B ? smem_desc_kmajor_sw128(b_addr + (k16 >> 2) * (N * 128) + (k16 & 3) * 32)
                                                : smem_desc_kmajor_noswz(b_addr + k16 * 256, B_LBO, B_SBO);
                const uint32_t acc = (ks > ks0 || k16 > 0) ? 1u : 0u;
                mma_ts(d_tmem, a_base + as * C::SLOT_COLS + kk * 8, bdesc, idesc_u, acc);
              }
              tc_commit(&ctl.a_empty[mg][as]);
            }
            __syncwarp();
            if (++as == NSLOT) { as = 0; apar ^= 1u; }
          }
          if (!ok) break;
          if (elect_one()) tc_commit(&ctl.b_empty[slot]);
          __syncwarp();
        }
        if (ok && elect_one()) tc_commit(&ctl.d_full[db]);
        __syncwarp();
        if (mg == 0 && lane == 0) MSK_TRD(1, tri, 2);
      }
      if (!ok) break;
    }
