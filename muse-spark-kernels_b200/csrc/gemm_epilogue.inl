// Role body of moe_gemm_kernel (included inside the kernel): epilogue, warps 4-7.
// Thread `row` reads TMEM lane `row` of both accumulator tiles of the unit. With K splits
// the raw accumulators go to partial[base unit][split][tile][row][N]; the thread block that
// draws the last ticket of a base unit sums the splits in index order and finishes.
    if (NDBUF > 1) {
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint32_t unit_i = 0, epi_par = 0;
    if (PHASE == 1) pdl_wait();  // y rows and the tables must not be touched before the previous grid is done
    bool ok = true;
    // bounded barrier over the 128 epilogue threads (a plain bar.sync could not time out)
    auto epi_sync = [&]() -> bool {
      mbar_arrive(&ctl.epi_bar);
      const bool r = mbar_wait(&ctl.epi_bar, epi_par, abortw);
      epi_par ^= 1u;
      return r;
    };
    for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++unit_i) {
      const UnitInfo ui = decode_unit(u, tile_start, p, N);
      const uint32_t db = unit_i % NDBUF, duse = unit_i / NDBUF;
      if (!mbar_wait(&ctl.d_full[db], duse & 1u, abortw)) { ok = false; break; }
      tc_fence_after();
      if (tid == 128) { if (unit_i == 0) MSK_TR(TR_FIRST_DFULL); MSK_TR(TR_LAST_DFULL); }
      const uint32_t d_tmem = tmem + lane_base + db * (2 * N);
      const float gsc = p.gs[ui.expert];
      const int base_unit = ui.tile * p.n_pairs + ui.pair;
      const size_t part_stride = static_cast<size_t>(2) * 128 * N;  // floats per (base unit, split)
      bool finish = true;
      if (p.splits > 1) {
        float* part = p.partial + (static_cast<size_t>(base_unit) * p.splits + ui.split) * part_stride;
#pragma unroll
        for (int t2 = 0; t2 < 2; ++t2) {
          float* dst = part + (static_cast<size_t>(t2) * 128 + row) * N;
#pragma unroll
          for (int c0 = 0; c0 < N; c0 += 16) {
            uint32_t r[16];
            tmem_ld16(d_tmem + t2 * N + c0, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; j += 4)
              *reinterpret_cast<uint4*>(dst + c0 + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
          }
        }
        // the accumulators are in memory: the MMA warp may reuse the buffer
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.d_empty[db]);
        __threadfence();
        if (!epi_sync()) { ok = false; break; }
        if (tid == 128) {
          const int old = atomicAdd(&p.tickets[base_unit], 1);
          const int last = (old == p.splits - 1) ? 1 : 0;
          if (last) p.tickets[base_unit] = 0;  // leave the workspace launch-ready
          __threadfence();
          ctl.last_flag = last;
        }
        if (!epi_sync()) { ok = false; break; }
        finish = ctl.last_flag != 0;
        if (!epi_sync()) { ok = false; break; }  // last_flag is rewritten by the next unit
      }
      if (finish) {
        const float* part0 = p.partial + static_cast<size_t>(base_unit) * p.splits * part_stride;
        if (PHASE == 0) {
          __half* outp = static_cast<__half*>(p.outp);
          const int col = ui.pair * 128 + row;
          for (int c0 = 0; c0 < N; c0 += 8) {
            if (c0 >= ui.rows) break;
            float ga[8], up[8];
            if (p.splits > 1) {
#pragma unroll
              for (int j = 0; j < 8; ++j) { ga[j] = 0.f; up[j] = 0.f; }
              for (int s = 0; s < p.splits; ++s) {
                const float* ps = part0 + s * part_stride;
                const float4* pg = reinterpret_cast<const float4*>(ps + static_cast<size_t>(row) * N + c0);
                const float4* pu = reinterpret_cast<const float4*>(ps + (128 + static_cast<size_t>(row)) * N + c0);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                  const float4 a = __ldcg(pg + j), b = __ldcg(pu + j);
                  ga[4 * j] += a.x; ga[4 * j + 1] += a.y; ga[4 * j + 2] += a.z; ga[4 * j + 3] += a.w;
                  up[4 * j] += b.x; up[4 * j + 1] += b.y; up[4 * j + 2] += b.z; up[4 * j + 3] += b.w;
                }
              }
            } else {
              uint32_t r0[8], r1[8];
              tmem_ld8(d_tmem + c0, r0);
              tmem_ld8(d_tmem + N + c0, r1);
              tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < 8; ++j) { ga[j] = __uint_as_float(r0[j]); up[j] = __uint_as_float(r1[j]); }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int n = c0 + j;
              if (n < ui.rows) {
                const float v = silu_f(ga[j] * gsc) * (up[j] * gsc);
                outp[static_cast<size_t>(ui.row0 + n) * p.out_ld + col] = inter_value(v);
              }
            }
          }
        } else {
          float* outp = static_cast<float*>(p.outp);
#pragma unroll
          for (int t2 = 0; t2 < 2; ++t2) {
            const int col = (2 * ui.pair + t2) * 128 + row;
            float osc = gsc;
            if (p.post_norm_w != nullptr) osc *= 1.0f + __bfloat162float(p.post_norm_w[col]);
            for (int c0 = 0; c0 < N; c0 += 8) {
              if (c0 >= ui.rows) break;
              float acc[8];
              if (p.splits > 1) {
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                for (int s = 0; s < p.splits; ++s) {
                  const float* ps = part0 + s * part_stride;
                  const float4* pp =
                      reinterpret_cast<const float4*>(ps + (static_cast<size_t>(t2) * 128 + row) * N + c0);
#pragma unroll
                  for (int j = 0; j < 2; ++j) {
                    const float4 a = __ldcg(pp + j);
                    acc[4 * j] += a.x; acc[4 * j + 1] += a.y; acc[4 * j + 2] += a.z; acc[4 * j + 3] += a.w;
                  }
                }
              } else {
                uint32_t r[8];
                tmem_ld8(d_tmem + t2 * N + c0, r);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = __uint_as_float(r[j]);
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int n = c0 + j;
                if (n < ui.rows) outp[static_cast<size_t>(ui.row0 + n) * p.out_ld + col] = acc[j] * osc;
              }
            }
          }
        }
      }
      if (p.splits == 1) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.d_empty[db]);
      }
      if (tid == 128 && unit_i == 0) MSK_TR(TR_FIRST_EPI_DONE);
    }
    }
