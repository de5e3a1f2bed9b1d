// Role body of moe_gemm_kernel (included inside the kernel): activation gather, warp 2.
// Copies the token rows of the piece (x rows through the permutation for phase 0, sorted inter
// rows for phase 1) with 16-byte cp.async into the K-major core-matrix layout of the B operand:
// element (n, k) at (n/8)*B_SBO + (k/8)*B_LBO + (n%8)*16 + (k%8)*2. Eight lanes write one
// 128-byte core matrix, so shared-memory writes are conflict free. A stage is published a few
// stages late, once its copies have landed and a proxy fence has ordered them before the
// tensor core's reads.
    if (!TMA_B) {
    constexpr int NG = N / 8;   // 8-token groups of the tile
    const int n_sub = lane & 7, c_sub = lane >> 3;  // token within an 8-group, chunk within a 4-chunk group
    // A stage is published GLAG stages after it was issued, so the loop never waits for the
    // copies it has just started (one stage of lag made every iteration a full memory latency).
    constexpr int GLAG = NST >= 5 ? 3 : (NST >= 4 ? 2 : 1);
    uint32_t it = 0, signalled = 0;
    int tri = 0;
    (void)tri;
    const uint64_t keep = policy_evict_last();  // token rows are re-read by every pair of the expert
    bool ok = true;
    // everything issued so far has landed: publish it
    auto drain = [&]() {
      if (signalled < it) {
        cp_async_wait<0>();
        fence_proxy_async_smem();
        __syncwarp();
        for (; signalled < it; ++signalled)
          if (lane == 0) mbar_arrive(&ctl.b_full[signalled % NST]);
        if (lane == 0) MSK_TRD(4, tri, 5);
      }
    };
    MSK_PHASES {
      MSK_PHASE_SETUP;
      // What the rows of this phase wait for. Two launches: inter is written by the gate/up GEMM, and the
      // F16 token rows, when the gate/up kernel routes itself, by the row-copy kernel launched in front
      // of it. One launch: every CTA's slice of the F16 rows (stage 1 of the grid counter), then every
      // CTA's rows of inter (stage 2).
      // (the wait itself sits below, in front of the first copy of the phase, after the addresses of
      // that copy have been worked out)
      bool must_wait = FUSED && phase == 0;
      int last_tile = -1;
      const bool per_tile = FUSED || (MODE == 1 && p.handover != 0);   // inter is handed over tile by tile
      if (!FUSED && ((MODE == 1 && !per_tile) || routed_here)) pdl_wait();
      const size_t act_ld = static_cast<size_t>(pp.K);
      while (ok && pieces.next(base, ks0, ks1)) {
        const UnitInfo ui = decode_unit(base, tile_start, pp.n_pairs, p.nloc, N);
        // source row of token n = ng*8 + n_sub, for every 8-group ng
        const __half* src[NG];
#pragma unroll
        for (int ng = 0; ng < NG; ++ng) {
          const int n = ng * 8 + n_sub;
          src[ng] = nullptr;
          if (n < ui.rows) {
            const int r = ui.row0 + n;
            size_t row = static_cast<size_t>(r);
            if (phase == 0) row = static_cast<size_t>((routed_here ? static_cast<int>(ctl.perm8[r]) : p.perm[r]) / p.top_k);
            src[ng] = static_cast<const __half*>(pp.act) + row * act_ld;
          }
        }
        bool first_piece = false;
        if (per_tile && (must_wait || (phase == 1 && ui.tile != last_tile))) {
          // phase 0: every CTA's slice of the F16 token rows; phase 1: the gate/up units of this token
          // tile. Everything issued so far is handed over first, so that the MMA warps never starve on
          // copies that have long landed.
          drain();
          int go = 1;
          if (lane == 0) {
            go = phase == 0 ? grid_counter_wait(p.grid_bar, n_ctas, abortw)
                            : grid_counter_wait(p.tile_done + ui.tile, static_cast<unsigned>(p.ph[0].n_pairs), abortw);
          }
          go = __shfl_sync(0xffffffffu, go, 0);
          if (!go) { ok = false; break; }
          if (lane == 0) MSK_TRD(4, tri, 1 + phase);
          first_piece = must_wait || phase == 1;
          must_wait = false;
          last_tile = ui.tile;
        }
        if (per_tile && phase == 1 && lane == 0) {
          // every down unit of the tile reports that it has seen the count complete; the last one puts both
          // counters back to zero for the next launch
          const unsigned seen = atomicAdd(p.tile_seen + ui.tile, 1u);
          if (seen == static_cast<unsigned>(pp.n_pairs) - 1u) {
            atomicExch(p.tile_done + ui.tile, 0u);
            atomicExch(p.tile_seen + ui.tile, 0u);
          }
        }
        for (int ks = ks0; ks < ks1; ++ks, ++it) {
          const uint32_t slot = it % NST, par = (it / NST) & 1u;
#ifdef MSK_TRACE_DETAIL
          if (lane == 0 && !mbar_test(&ctl.b_empty[slot], par ^ 1u)) MSK_TRD(4, tri, 6);   // B slot still in use
#endif
          if (!MSK_WAIT(&ctl.b_empty[slot], par ^ 1u, abortw)) { ok = false; break; }
          uint8_t* dstB = ring + slot * C::STAGE_BYTES + 2 * TILE_BYTES;
#pragma unroll
          for (int ng = 0; ng < NG; ++ng) {
            const bool valid = src[ng] != nullptr;
            const __half* s = valid ? src[ng] + static_cast<size_t>(ks) * KS : static_cast<const __half*>(pp.act);
#pragma unroll
            for (int cg = 0; cg < 8; ++cg) {
              const int chunk = cg * 4 + c_sub;
              cp_async16_hint(dstB + ng * B_SBO + chunk * B_LBO + n_sub * 16, s + chunk * 8, valid, keep);
            }
          }
          cp_async_commit();
          if (lane == 0) MSK_TRD(4, tri, 3);
          if (it + 1 - signalled > GLAG) {
            cp_async_wait<GLAG>();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl.b_full[signalled % NST]);
            ++signalled;
            if (lane == 0) MSK_TRD(4, tri, 4);
          }
        }
        // right behind a wait on other CTAs the MMA warps may stand idle: hand the piece over as soon as it
        // has landed instead of a few stages late
        if (ok && first_piece) drain();
      }
      if (!ok) break;
      // a CTA without work in this phase still takes part in nothing it has to wait for
    }
    drain();
    }
