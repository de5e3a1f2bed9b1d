// Role body of moe_gemm_kernel (included inside the kernel): dequant, warps 8-23.
// Warp = (K half kh, tile g, lane quarter). Thread `row` of a quarter owns one weight row of
// tile g. Per K stage the warps of half kh fill A slots kh and kh+2 (64 K each): two 16-byte
// code chunks and four scale bytes -> 32 BF16x2 registers -> two tcgen05.st. A slot is
// handed to the MMA warp one slot late (`retire`), so the store latency hides behind the
// decode of the following slot.
    const int didx = warp - 8;
    const int g = (didx >> 2) & 1;
    const int kh = didx >> 3;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t a_tmem = tmem + lane_base + C::A_BASE + g * C::A_GROUP_COLS;
    const uint32_t lut_s = smem_u32(lut);
    uint32_t it = 0;
    int tri = 0;
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
    for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
      const UnitInfo ui = decode_unit(u, tile_start, p, N);
      const int ks0 = ui.split * per_split, ks1 = min(nst_total, ks0 + per_split);
      for (int ks = ks0; ks < ks1 && ok; ++ks, ++it) {
        const uint32_t slot = it % NST, par = (it / NST) & 1u;
        if (!mbar_wait(&ctl.raw_full[slot], par, abortw)) { ok = false; break; }
        if (it == 0 && tid == 256) MSK_TR(TR_FIRST_RAW);
        if (tid == 256) MSK_TRD(0, tri, 1);
        const uint32_t tile = smem_u32(ring + slot * C::STAGE_BYTES + g * TILE_BYTES);
        uint32_t sfa[4];
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(sfa[0]), "=r"(sfa[1]), "=r"(sfa[2]), "=r"(sfa[3])
                     : "r"(tile + TILE_CODE_BYTES + row * 16));
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int sl = 2 * i + kh;             // 64 K per A slot = two 32-K chunks = four scale blocks
          const uint32_t sc = it * 4u + sl;
          uint32_t o[32];
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int chunk = sl * 2 + c;
            uint32_t q[4];
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3])
                         : "r"(tile + (chunk * 128 + row) * 16));
            const uint32_t sw = (chunk & 1) ? (sfa[chunk >> 1] >> 16) : sfa[chunk >> 1];
#ifdef MSK_EXP_ARITH_SCALE
            const uint32_t t16 = ((prmt(sw, 0u, 0x4140u) & 0x007F007Fu) << 4) + 0x5C005C00u;
            const uint32_t s0 = prmt(t16, 0u, 0x1010u), s1 = prmt(t16, 0u, 0x3232u);
#else
            const uint32_t s0 = lds32(lut_s + ((sw << 2) & 0x3FCu)), s1 = lds32(lut_s + ((sw >> 6) & 0x3FCu));
#endif
            uint32_t* oc = o + c * 16;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
#ifdef MSK_EXP_NO_ALU
              oc[4 * w + 0] = q[w]; oc[4 * w + 1] = q[w] ^ s0; oc[4 * w + 2] = q[w] + s1; oc[4 * w + 3] = q[w] | 1u;
#else
              uint32_t r0, r1, r2, r3;
              decode_codes(q[w], r0, r1, r2, r3);
              const uint32_t s = w < 2 ? s0 : s1;
              oc[4 * w + 0] = hmul2_bf16(r0, s);
              oc[4 * w + 1] = hmul2_bf16(r1, s);
              oc[4 * w + 2] = hmul2_bf16(r2, s);
              oc[4 * w + 3] = hmul2_bf16(r3, s);
#endif
            }
          }
          if (tid == 256) MSK_TRD(0, tri, 2);
          if (pending) retire();
          const uint32_t as = sc % NSLOT, apar = (sc / NSLOT) & 1u;
          if (!mbar_wait(&ctl.a_empty[as], apar ^ 1u, abortw)) { ok = false; break; }
          tc_fence_after();
          if (tid == 256) MSK_TRD(0, tri, 3);
          tmem_st32(a_tmem + as * 32, o);
          pending = true;
          pending_slot = as;
          if (sc == 0 && tid == 256) MSK_TR(TR_FIRST_AFULL);
        }
        if (!ok) break;
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.raw_empty[slot]);
      }
      if (!ok) break;
      if (pending) retire();  // the accumulators need every slot of the unit
    }
