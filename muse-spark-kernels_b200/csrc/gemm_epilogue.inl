// Role body of moe_gemm_kernel (included inside the kernel): epilogue, warps 4-7.
// Thread `row` reads TMEM lane `row` of both accumulator tiles of the piece. A whole unit goes
// straight from TMEM through the epilogue math to global memory. A piece of a cut unit (flat
// shares) stores its raw accumulators to this CTA's slot of the partial buffer and takes the
// unit's ticket; the CTA that draws the last ticket sums the pieces in ascending K order and
// finishes the unit.
    if (NDBUF > 1) {
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint32_t unit_i = 0, epi_par = 0;
    if (MODE == 1) pdl_wait();  // y rows and tickets must not be touched before the previous grid is done
    bool ok = true;
    // bounded barrier over the 128 epilogue threads (a plain bar.sync could not time out)
    auto epi_sync = [&]() -> bool {
      mbar_arrive(&ctl.epi_bar);
      const bool r = mbar_wait(&ctl.epi_bar, epi_par, abortw);
      epi_par ^= 1u;
      return r;
    };
    constexpr size_t part_stride = static_cast<size_t>(2) * 128 * N;  // floats per piece
    MSK_PHASES {
      MSK_PHASE_SETUP;
      const long long items = static_cast<long long>(n_base) * nst_total;
      for (; ok && pieces.next(base, ks0, ks1); ++unit_i) {
        const UnitInfo ui = decode_unit(base, tile_start, pp.n_pairs, p.nloc, N);
        const uint32_t db = unit_i % NDBUF, duse = unit_i / NDBUF;
        if (!mbar_wait(&ctl.d_full[db], duse & 1u, abortw)) { ok = false; break; }
        tc_fence_after();
        if (tid == 128) { if (unit_i == 0) MSK_TR(TR_FIRST_DFULL); MSK_TR(TR_LAST_DFULL); }
        const uint32_t d_tmem = tmem + lane_base + db * (2 * N);
        const float gsc = pp.gs[ui.expert];
        const bool whole = ks0 == 0 && ks1 == nst_total;
        bool finish = true;
        int c_first = 0, c_last = 0;
        if (!whole) {
          float* part = pp.partial + static_cast<size_t>(piece_slot(static_cast<int>(blockIdx.x), ks0 == 0)) * part_stride;
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
          // the shares that hold a piece of this unit: first and last owner of its K stages
          const long long b0 = static_cast<long long>(base) * nst_total;
          c_first = share_owner(items, static_cast<int>(n_ctas), b0);
          c_last = share_owner(items, static_cast<int>(n_ctas), b0 + nst_total - 1);
          if (tid == 128) {
            // pieces of the unit: the shares from c_first to c_last that hold anything at all (with fewer
            // items than CTAs some shares are empty)
            int n_pieces = 0;
            for (int c = c_first; c <= c_last; ++c)
              n_pieces += share_begin(items, static_cast<int>(n_ctas), c + 1) > share_begin(items, static_cast<int>(n_ctas), c) ? 1 : 0;
            const int old = atomicAdd(&pp.tickets[base], 1);
            const int last = (old == n_pieces - 1) ? 1 : 0;
            if (last) pp.tickets[base] = 0;  // leave the workspace launch-ready
            __threadfence();
            ctl.last_flag = last;
          }
          if (!epi_sync()) { ok = false; break; }
          finish = ctl.last_flag != 0;
          if (!epi_sync()) { ok = false; break; }  // last_flag is rewritten by the next piece
        }
        if (finish) {
          const long long b0 = static_cast<long long>(base) * nst_total;
          if (phase == 0) {
            __half* outp = static_cast<__half*>(pp.outp);
            const int col = ui.pair * 128 + row;
            for (int c0 = 0; c0 < N; c0 += 8) {
              if (c0 >= ui.rows) break;
              float ga[8], up[8];
              if (!whole) {
#pragma unroll
                for (int j = 0; j < 8; ++j) { ga[j] = 0.f; up[j] = 0.f; }
                for (int c = c_first; c <= c_last; ++c) {   // ascending K
                  const long long sb = share_begin(items, static_cast<int>(n_ctas), c);
                  if (share_begin(items, static_cast<int>(n_ctas), c + 1) <= sb) continue;  // an empty share
                  const float* ps = pp.partial + static_cast<size_t>(piece_slot(c, sb <= b0)) * part_stride;
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
                  outp[static_cast<size_t>(ui.row0 + n) * pp.out_ld + col] = inter_value(v);
                }
              }
            }
          } else {
            float* outp = static_cast<float*>(pp.outp);
#pragma unroll
            for (int t2 = 0; t2 < 2; ++t2) {
              const int col = (2 * ui.pair + t2) * 128 + row;
              float osc = gsc;
              if (p.post_norm_w != nullptr) osc *= 1.0f + __bfloat162float(p.post_norm_w[col]);
              for (int c0 = 0; c0 < N; c0 += 8) {
                if (c0 >= ui.rows) break;
                float acc[8];
                if (!whole) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                  for (int c = c_first; c <= c_last; ++c) {   // ascending K
                    const long long sb = share_begin(items, static_cast<int>(n_ctas), c);
                    if (share_begin(items, static_cast<int>(n_ctas), c + 1) <= sb) continue;  // an empty share
                    const float* ps = pp.partial + static_cast<size_t>(piece_slot(c, sb <= b0)) * part_stride;
                    const float4* pq = reinterpret_cast<const float4*>(ps + (static_cast<size_t>(t2) * 128 + row) * N + c0);
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                      const float4 a = __ldcg(pq + j);
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
                  if (n < ui.rows) outp[static_cast<size_t>(ui.row0 + n) * pp.out_ld + col] = acc[j] * osc;
                }
              }
            }
          }
        }
        if (whole) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl.d_empty[db]);
        }
        if (fold && phase == 1) {
          // Token tickets: a base unit that has just been finished counts once for every token that has a
          // row in it. The CTA that brings a token's ticket to (its local routes) x (pairs) has seen the
          // token's last unit and puts it on its list for the folded combine.
          __threadfence();
          if (!epi_sync()) { ok = false; break; }
          const int j = tid - 128;
          if (finish && j < ui.rows) {
            const int t = static_cast<int>(ctl.perm8[ui.row0 + j]) / p.top_k;
            const int want = static_cast<int>(ctl.klocal[t]) * pp.n_pairs;
            const int old = atomicAdd(&p.tok_tickets[t], 1);
            if (old == want - 1) {
              p.tok_tickets[t] = 0;  // launch-ready again
              __threadfence();
              const int at = atomicAdd(&ctl.fin_n, 1);
              if (at < FOLD_MAX_TOKENS) ctl.fin_tok[at] = static_cast<uint8_t>(t);
            }
          }
        }
        if (tid == 128 && unit_i == 0) MSK_TR(TR_FIRST_EPI_DONE);
      }
      if (!ok) break;
      if (FUSED && phase == 0) {
        // stage 2 of the grid counter: every row of inter this CTA had to write is in memory
        __threadfence();
        if (!epi_sync()) { ok = false; break; }
        if (tid == 128) atomicAdd(p.grid_bar, 1u);
      }
    }
    }
