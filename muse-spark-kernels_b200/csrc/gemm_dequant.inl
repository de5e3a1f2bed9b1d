// Role body of moe_gemm_kernel (included inside the kernel): dequant, warps 8-23.
// Warp = (K half kh, tile g, lane quarter). Thread `row` of a quarter owns one weight row of
// tile g. Per K stage the warps of half kh fill one A slot (128 K): four 16-byte code chunks
// and eight scale bytes -> 4 x 16 BF16x2 registers -> four tcgen05.st, each issued right after
// its chunk is decoded. With three slots per tile a slot is handed to the MMA warp (`retire`) after
// the first chunk of the following slot has been decoded, so the store latency hides behind it; with
// two slots right behind its stores (see below). Slots of half the size (64 K, twice as many
// hand-overs) were measured too: 10 - 20 % slower at every size, the hand-over itself is what costs.
    const int didx = warp - 8;
    const int g = (didx >> 2) & 1;
    const int kh = didx >> 3;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t a_tmem = tmem + lane_base + C::A_BASE + g * C::A_GROUP_COLS;
    uint32_t it = 0;
    int tri = 0;
    uint32_t as = kh, apar = 0;  // ring slot of this warp's next K half and its phase parity
    bool ok = true;
    bool pending = false;      // stores of the previous slot issued, slot not yet handed over
    uint32_t pending_slot = 0;
    auto retire = [&]() {
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.a_full[g][pending_slot]);
      pending = false;
    };
    uint32_t unit_i = 0;
    // Single accumulator buffer (the 128-token tile): the main loop cannot go on until the accumulators
    // are drained, and the sixteen dequant warps drain them together (the four warps of a lane quarter
    // split the columns). The drain of a unit is put off until this warp has decoded the first stage
    // of the next unit into the A slots, which are free by then: when the drain ends, the MMA warps find
    // their operands ready, and the bubble between two units is the drain alone, not the drain plus
    // a refill of the decode pipeline.
    bool owe_drain = false;
    UnitInfo owed_ui;
    uint32_t owed_unit_i = 0;
    MSK_PHASES {
      MSK_PHASE_SETUP;
      auto drain = [&]() -> bool {
        if (!MSK_WAIT(&ctl.d_full[0], owed_unit_i & 1u, abortw)) return false;
        tc_fence_after();
        if (tid == 256) { if (owed_unit_i == 0) MSK_TR(TR_FIRST_DFULL); MSK_TR(TR_LAST_DFULL); }
        if (phase == 0) {
          const int part = kh * 2 + g;  // 0..3: a quarter of the token columns, gate and up of this lane
          epilogue_columns<N>(p, pp, phase, owed_ui, tmem + lane_base, row, part * (N / 4), (part + 1) * (N / 4), 0);
        } else {
          epilogue_columns<N>(p, pp, phase, owed_ui, tmem + lane_base, row, kh * (N / 2), (kh + 1) * (N / 2), g);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.d_empty[0]);
        if (tid == 256 && owed_unit_i == 0) MSK_TR(TR_FIRST_EPI_DONE);
        owe_drain = false;
        return true;
      };
      for (; ok && pieces.next(base, ks0, ks1); ++unit_i) {
        const UnitInfo ui = decode_unit(base, tile_start, pp.n_pairs, p.nloc, N);
        for (int ks = ks0; ks < ks1 && ok; ++ks, ++it) {
          const uint32_t slot = it % NST, par = (it / NST) & 1u;
#ifdef MSK_TRACE_DETAIL
          // first and last dequant warp (roles 0 and 5): 1 the stage had landed before the warp asked for it, 3 it had not
          if (lane == 0 && (didx == 0 || didx == 15)) {
            if (mbar_test(&ctl.raw_full[slot], par)) MSK_TRD(didx ? 5 : 0, tri, 1);
            else MSK_TRD(didx ? 5 : 0, tri, 3);
          }
#endif
          if (!MSK_WAIT(&ctl.raw_full[slot], par, abortw)) { ok = false; break; }
          if (it == 0 && tid == 256) MSK_TR(TR_FIRST_RAW);
          if (lane == 0 && (didx == 0 || didx == 15)) MSK_TRD(didx ? 5 : 0, tri, 5);
          const uint32_t tile = smem_u32(ring + slot * C::STAGE_BYTES + g * TILE_BYTES);
          const uint32_t tile_row = tile + row * 16;
          uint32_t sfa[4];
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(sfa[0]), "=r"(sfa[1]), "=r"(sfa[2]), "=r"(sfa[3])
                       : "r"(tile + TILE_CODE_BYTES + row * 16));
          {
            // this warp's slot of the stage: K half kh = chunks 4*kh .. 4*kh+3
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const int chunk = kh * 4 + c;
              uint32_t q[4];
              asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3])
                           : "r"(tile_row + chunk * 2048));
              const uint32_t sfw = kh ? (c < 2 ? sfa[2] : sfa[3]) : (c < 2 ? sfa[0] : sfa[1]);
              uint32_t o[16];
              decode_chunk(q, (c & 1) ? (sfw >> 16) : sfw, o);
              if (c == 0) {
                // hand over the previous slot (its stores had the decode above to land), claim this one
                if (pending) retire();
#ifdef MSK_TRACE_DETAIL
                if (lane == 0 && (didx == 0 || didx == 15) && !mbar_test(&ctl.a_empty[g][as], apar ^ 1u))
                  MSK_TRD(didx ? 5 : 0, tri, 9);   // the A slot was not free yet
#endif
                if (!MSK_WAIT(&ctl.a_empty[g][as], apar ^ 1u, abortw)) { ok = false; break; }
                if (lane == 0 && (didx == 0 || didx == 15)) MSK_TRD(didx ? 5 : 0, tri, 6);
                tc_fence_after();
              }
              tmem_st16(a_tmem + as * C::SLOT_COLS + c * 16, o);
            }
            if (!ok) break;
            pending = true;
            pending_slot = as;
            // Two-slot rings (the wide token tiles): this K half's slot is refilled every stage, and the refill
            // has to wait until the MMAs of the stage before have drained it. Handing the slot over right
            // here, instead of behind the first decode of the next stage, lets those MMAs start a decode
            // earlier (8192 tokens: gate/up GEMM 1.47 -> 1.34 ms; 256 tokens 309 -> 300 us a step). With three
            // slots (the narrow tiles) it changes nothing, and the deferred hand-over hides the store latency.
            // (Letting both warp groups of a tile decode the same slot, so that a slot fills in half the time,
            // was measured on top of this: no change.)
            if (NSLOT == 2) retire();
            if (it == 0 && tid == 256) MSK_TR(TR_FIRST_AFULL);
            // the other K half takes the next ring slot; this warp's next one is two further
            as += 2;
            if (as >= NSLOT) { as -= NSLOT; apar ^= 1u; }
          }
          if (!ok) break;
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl.raw_empty[slot]);
          if (lane == 0 && (didx == 0 || didx == 15)) MSK_TRD(didx ? 5 : 0, tri, 7);
          if (NDBUF == 1 && owe_drain) {
            if (pending) retire();   // the first stage of this unit is ready for the MMA warps
            if (!drain()) { ok = false; break; }
          }
        }
        if (!ok) break;
        if (pending) retire();  // the accumulators need every slot of the piece
        if (NDBUF == 1) {
          owe_drain = true;
          owed_ui = ui;
          owed_unit_i = unit_i;
        }
      }
      if (ok && NDBUF == 1 && owe_drain && !drain()) ok = false;   // the last unit of the phase
      if (!ok) break;
    }
