// Role body of moe_gemm_kernel (included inside the kernel): weight producer, warp 0.
// One lane streams the two packed tiles of every K stage of every piece of this CTA into the
// shared-memory ring with 1-D bulk async copies that complete on the stage's mbarrier. With both
// phases in one launch the stream runs on from the last gate/up stage into the first down stage.
//
// The ring is the only look-ahead. Asking L2 for stages further ahead (cp.async.bulk.prefetch.L2 from
// this lane, 4 to 32 stages in front of the ring) was built and measured: every few-token point got
// slower (one token 46 -> 48 us at 8 stages, 64 tokens 262 -> 274 us), because the main loop does not
// wait for memory (with the weight copies left out altogether the steps take the same time) and each
// prefetch occupies the copy engine of the SM for as long as the copy it anticipates.
    if (lane == 0) {
      const uint64_t pol = p.evict_first ? policy_evict_first() : policy_evict_last();
      const uint64_t keep = policy_evict_last();  // token rows are re-read by every pair of the expert
      (void)keep;
      uint32_t it = 0;
      int tri = 0;
      bool ok = true;
      MSK_PHASES {
        MSK_PHASE_SETUP;
        while (ok && pieces.next(base, ks0, ks1)) {
          const UnitInfo ui = decode_unit(base, tile_start, pp.n_pairs, p.nloc, N);
          const size_t tile0 =
              (static_cast<size_t>(ui.expert) * (2 * pp.n_pairs) + 2 * ui.pair) * static_cast<size_t>(nst_total);
          const uint8_t* g0 = pp.w + tile0 * TILE_BYTES;
          const uint8_t* g1 = g0 + static_cast<size_t>(nst_total) * TILE_BYTES;
          for (int ks = ks0; ks < ks1; ++ks, ++it) {
            const uint32_t slot = it % NST, par = (it / NST) & 1u;
#ifdef MSK_TRACE_DETAIL
            if (!mbar_test(&ctl.raw_empty[slot], par ^ 1u)) MSK_TRD(2, tri, 2);   // ring slot still being read
#endif
            if (!MSK_WAIT(&ctl.raw_empty[slot], par ^ 1u, abortw)) { ok = false; break; }
            uint8_t* dst = ring + slot * C::STAGE_BYTES;
            mbar_arrive_expect_tx(&ctl.raw_full[slot], 2 * TILE_BYTES);
            bulk_g2s(dst, g0 + static_cast<size_t>(ks) * TILE_BYTES, TILE_BYTES, &ctl.raw_full[slot], pol);
            bulk_g2s(dst + TILE_BYTES, g1 + static_cast<size_t>(ks) * TILE_BYTES, TILE_BYTES, &ctl.raw_full[slot], pol);
            if (it == 0) MSK_TR(TR_FIRST_BULK);
            if (TMA_B) {
              // activation tile of the stage: four boxes of 64 K x N rows, rows row0.. of the sorted matrix.
              // (Fetching only the 32-row groups a tile's rows lie in, with a second tensor map of 64 x 32
              // boxes, halves the bytes of a sparsely filled tile and was slower: 256 tokens 351 against
              // 307 us. More copies per stage cost more than the bytes they save.)
              if (MODE == 1 && it == 0) pdl_wait();  // inter comes from the gate/up GEMM
              if (!MSK_WAIT(&ctl.b_empty[slot], par ^ 1u, abortw)) { ok = false; break; }
              uint8_t* dstB = dst + 2 * TILE_BYTES;
              mbar_arrive_expect_tx(&ctl.b_full[slot], C::B_STAGE_BYTES);
#pragma unroll
              for (int j = 0; j < 4; ++j)
                tma_load_2d(dstB + j * (N * 128), &p.tmap_act[phase], ks * KS + j * 64, ui.row0, &ctl.b_full[slot], keep);
            }
            MSK_TRD(2, tri, 1);
          }
        }
        if (!ok) break;
      }
      if (MODE == 0 && ok && p.ph[1].w != nullptr) {
        // This CTA's own weight stream has been issued. The down GEMM that follows is dealt the same way
        // over the same token tiles, so its CTA of this index will start on the stages named below: pull
        // the first ring-full of them into L2 now, while the pipeline here drains and the next kernel sets
        // up (the reference lets its last gate/up refills fetch the first down units,
        // muse_moe_w4a16/cuda/moe.cu:615-617, 2307-2318).
        const PhaseParams& nx = p.ph[1];
        const int nst2 = nx.K / KS;
        PieceIter pi = make_piece_iter(iter_mode, ctl.n_tiles * nx.n_pairs, nst2, static_cast<int>(blockIdx.x),
                                       static_cast<int>(n_ctas));
        int left = NST + 1, b2, k0, k1;
        while (left > 0 && pi.next(b2, k0, k1)) {
          const UnitInfo u2 = decode_unit(b2, tile_start, nx.n_pairs, p.nloc, N);
          const size_t t0 = (static_cast<size_t>(u2.expert) * (2 * nx.n_pairs) + 2 * u2.pair) * static_cast<size_t>(nst2);
          const int take = min(left, k1 - k0);
          prefetch_l2(nx.w + (t0 + k0) * TILE_BYTES, static_cast<uint32_t>(take) * TILE_BYTES);
          prefetch_l2(nx.w + (t0 + nst2 + k0) * TILE_BYTES, static_cast<uint32_t>(take) * TILE_BYTES);
          left -= take;
        }
      }
    }
