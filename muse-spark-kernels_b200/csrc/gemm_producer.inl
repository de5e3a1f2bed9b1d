// Role body of moe_gemm_kernel (included inside the kernel): weight producer, warp 0.
// One lane streams the two packed tiles of every K stage of every unit of this CTA into the
// shared-memory ring with 1-D bulk async copies that complete on the stage's mbarrier.
    if (lane == 0) {
      const uint64_t pol = p.evict_first ? policy_evict_first() : policy_evict_last();
      const uint64_t keep = policy_evict_last();  // token rows are re-read by every pair of the expert
      (void)keep;
      uint32_t it = 0;
      int tri = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
        const UnitInfo ui = decode_unit(u, tile_start, p, N);
        const int ks0 = ui.split * per_split, ks1 = min(nst_total, ks0 + per_split);
        const size_t tile0 =
            (static_cast<size_t>(ui.expert) * (2 * p.n_pairs) + 2 * ui.pair) * static_cast<size_t>(nst_total);
        const uint8_t* g0 = p.w + tile0 * TILE_BYTES;
        const uint8_t* g1 = g0 + static_cast<size_t>(nst_total) * TILE_BYTES;
        for (int ks = ks0; ks < ks1; ++ks, ++it) {
          const uint32_t slot = it % NST, par = (it / NST) & 1u;
          if (!mbar_wait(&ctl.raw_empty[slot], par ^ 1u, abortw)) { ok = false; break; }
          uint8_t* dst = ring + slot * C::STAGE_BYTES;
          mbar_arrive_expect_tx(&ctl.raw_full[slot], 2 * TILE_BYTES);
          bulk_g2s(dst, g0 + static_cast<size_t>(ks) * TILE_BYTES, TILE_BYTES, &ctl.raw_full[slot], pol);
          bulk_g2s(dst + TILE_BYTES, g1 + static_cast<size_t>(ks) * TILE_BYTES, TILE_BYTES, &ctl.raw_full[slot], pol);
          if (it == 0) MSK_TR(TR_FIRST_BULK);
          if (C::TMA_B) {
            // activation tile of the stage: four boxes of 64 K x N rows, rows row0.. of the sorted matrix
            if (PHASE == 1 && it == 0) pdl_wait();  // inter comes from the gate/up GEMM
            if (!mbar_wait(&ctl.b_empty[slot], par ^ 1u, abortw)) { ok = false; break; }
            uint8_t* dstB = dst + 2 * TILE_BYTES;
            mbar_arrive_expect_tx(&ctl.b_full[slot], C::B_STAGE_BYTES);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tma_load_2d(dstB + j * (N * 128), &p.tmap_act, ks * KS + j * 64, ui.row0, &ctl.b_full[slot], keep);
          }
          MSK_TRD(2, tri, 1);
        }
      }
    }
