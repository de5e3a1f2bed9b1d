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
    int tri = 0;
    (void)tri;
    // y rows and tickets must not be touched before the previous grid is done; with the per-tile hand-over a
    // unit gets here only after its tile's gate/up units have finished, which is later than that grid's own wait
    if (MODE == 1 && !p.handover) pdl_wait();
    bool ok = true;
    // bounded barrier over the 128 epilogue threads (a plain bar.sync could not time out)
    auto epi_sync = [&]() -> bool {
      mbar_arrive(&ctl.epi_bar);
      const bool r = mbar_wait_short(&ctl.epi_bar, epi_par, abortw);
      epi_par ^= 1u;
      return r;
    };
    constexpr size_t part_stride = static_cast<size_t>(2) * 128 * N;  // floats per piece
    MSK_PHASES {
      MSK_PHASE_SETUP;
      const int items = (n_base - tail_base) * nst_total;   // the flat tail, where units are cut
      for (; ok && pieces.next(base, ks0, ks1); ++unit_i) {
        const UnitInfo ui = decode_unit(base, tile_start, pp.n_pairs, p.nloc, N);
        const uint32_t db = unit_i % NDBUF, duse = unit_i / NDBUF;
        if (!MSK_WAIT(&ctl.d_full[db], duse & 1u, abortw)) { ok = false; break; }
        tc_fence_after();
        if (tid == 128) { if (unit_i == 0) MSK_TR(TR_FIRST_DFULL); MSK_TR(TR_LAST_DFULL); MSK_TRD(3, tri, 1); }
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
          if (tid == 128) MSK_TRD(3, tri, 2);
          if (!epi_sync()) { ok = false; break; }
          // the shares that hold a piece of this unit: first and last owner of its K stages
          const int b0 = (base - tail_base) * nst_total;
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
            ctl.last_flag[unit_i & 1u] = last;   // two words in turn: the next piece writes the other one
          }
          if (tid == 128) MSK_TRD(3, tri, 3);
          if (!epi_sync()) { ok = false; break; }
          finish = ctl.last_flag[unit_i & 1u] != 0;
          if (tid == 128) MSK_TRD(3, tri, 4);
        }
        if (finish) {
          // (a cut unit: the pieces' partial accumulators are summed in ascending K order; plain loops on
          // purpose: this path runs once or twice per launch from a cold instruction cache, where every
          // extra line of code costs more than the loads it could overlap)
          const int b0 = (base - tail_base) * nst_total;
          const int col0 = phase == 0 ? ui.pair * 128 + row : (2 * ui.pair) * 128 + row;
          float osc0 = gsc, osc1 = gsc;
          if (phase == 1 && p.post_norm_w != nullptr) {
            osc0 *= 1.0f + __bfloat162float(p.post_norm_w[col0]);
            osc1 *= 1.0f + __bfloat162float(p.post_norm_w[col0 + 128]);
          }
          for (int c0 = 0; c0 < N; c0 += 8) {
            if (c0 >= ui.rows) break;
            float a0[8], a1[8];   // tile 0 (gate, or the even row tile) and tile 1 (up, or the odd one)
            if (!whole) {
#pragma unroll
              for (int j = 0; j < 8; ++j) { a0[j] = 0.f; a1[j] = 0.f; }
#pragma unroll 1
              for (int c = c_first; c <= c_last; ++c) {
                const int sb = share_begin(items, static_cast<int>(n_ctas), c);
                if (share_begin(items, static_cast<int>(n_ctas), c + 1) <= sb) continue;  // an empty share
                const float* ps = pp.partial + static_cast<size_t>(piece_slot(c, sb <= b0)) * part_stride;
                const float4* q0 = reinterpret_cast<const float4*>(ps + static_cast<size_t>(row) * N + c0);
                const float4* q1 = reinterpret_cast<const float4*>(ps + (128 + static_cast<size_t>(row)) * N + c0);
                const float4 x0 = __ldcg(q0), x1 = __ldcg(q0 + 1), y0 = __ldcg(q1), y1 = __ldcg(q1 + 1);
                a0[0] += x0.x; a0[1] += x0.y; a0[2] += x0.z; a0[3] += x0.w;
                a0[4] += x1.x; a0[5] += x1.y; a0[6] += x1.z; a0[7] += x1.w;
                a1[0] += y0.x; a1[1] += y0.y; a1[2] += y0.z; a1[3] += y0.w;
                a1[4] += y1.x; a1[5] += y1.y; a1[6] += y1.z; a1[7] += y1.w;
              }
            } else {
              uint32_t r0[8], r1[8];
              tmem_ld8(d_tmem + c0, r0);
              tmem_ld8(d_tmem + N + c0, r1);
              tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < 8; ++j) { a0[j] = __uint_as_float(r0[j]); a1[j] = __uint_as_float(r1[j]); }
            }
            if (phase == 0) {
              __half* outp = static_cast<__half*>(pp.outp);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int n = c0 + j;
                if (n < ui.rows) {
                  const float v = silu_f(a0[j] * gsc) * (a1[j] * gsc);
                  outp[static_cast<size_t>(ui.row0 + n) * pp.out_ld + col0] = inter_value(v);
                }
              }
            } else {
              float* outp = static_cast<float*>(pp.outp);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int n = c0 + j;
                if (n < ui.rows) {
                  float* orow = outp + static_cast<size_t>(ui.row0 + n) * pp.out_ld + col0;
                  orow[0] = a0[j] * osc0;
                  orow[128] = a1[j] * osc1;
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
        if (tid == 128) MSK_TRD(3, tri, 5);
        if ((FUSED || p.handover) && phase == 0) {
          // this unit's columns of inter are complete; count it for its token tile, whose down units (the
          // second phase of this launch, or the down GEMM launched behind it) wait for the count to reach
          // the number of gate/up pairs
          __threadfence();
          if (!epi_sync()) { ok = false; break; }
          if (finish && tid == 128) { atomicAdd(p.tile_done + ui.tile, 1u); MSK_TRD(3, tri, 7); }
        }
        if (fold && phase == 1) {
          // Tickets: a base unit that has just been finished counts once for every token that has a row in
          // it. With the post-expert norm a token can only be combined when all of its rows are complete
          // (the norm needs whole rows): one ticket per token, target (local routes) x (pairs); the CTA
          // that draws the last one puts the token on its list for the folded combine at the end of the
          // kernel. Without the norm the 256 output columns of this pair only need the same columns of the
          // token's other rows: one ticket per (token, pair), target (local routes), and the epilogue
          // threads of the CTA that draws the last one combine those columns right here.
          __threadfence();
          if (!epi_sync()) { ok = false; break; }
          const int j = tid - 128;
          const bool by_column = p.fold == 2;
          if (finish && j < ui.rows) {
            const int t = static_cast<int>(ctl.perm8[ui.row0 + j]) / p.top_k;
            const int want = by_column ? static_cast<int>(ctl.klocal[t]) : static_cast<int>(ctl.klocal[t]) * pp.n_pairs;
            int32_t* ticket = p.tok_tickets + (by_column ? t * pp.n_pairs + ui.pair : t);
            const int old = atomicAdd(ticket, 1);
            if (old == want - 1) {
              *ticket = 0;  // launch-ready again
              __threadfence();
              const int at = atomicAdd(&ctl.fin_n, 1);
              if (at < FOLD_MAX_TOKENS) ctl.fin_tok[at] = static_cast<uint8_t>(t);
            }
          }
          if (tid == 128) MSK_TRD(3, tri, 6);
          if (by_column) {
            if (!epi_sync()) { ok = false; break; }
            const int nf = finish ? ctl.fin_n : 0;
            const int H = pp.out_ld, col0 = (2 * ui.pair) * 128 + row;
            const float* yb = static_cast<const float*>(pp.outp);
#pragma unroll 1
            for (int f = 0; f < nf; ++f) {
              const int t = ctl.fin_tok[f];
              // lane s fetches slot s of the token; the sums below run in slot order
              const int qv = lane < p.top_k ? __ldcg(p.inv + t * p.top_k + lane) : -1;
              const float wv = lane < p.top_k ? __ldcg(p.tw + t * p.top_k + lane) : 0.f;
              float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
              for (int sl = 0; sl < p.top_k; ++sl) {
                const int q = __shfl_sync(0xffffffffu, qv, sl);
                const float w = __shfl_sync(0xffffffffu, wv, sl);
                if (q >= 0) {
                  const float* yr = yb + static_cast<size_t>(q) * H + col0;
                  a0 += __ldcg(yr) * w;
                  a1 += __ldcg(yr + 128) * w;
                }
              }
              __nv_bfloat16* orow = p.out + static_cast<size_t>(t) * H + col0;
              orow[0] = __float2bfloat16_rn(a0);
              orow[128] = __float2bfloat16_rn(a1);
            }
            if (!epi_sync()) { ok = false; break; }   // the list is read by all before it is emptied
            if (tid == 128) ctl.fin_n = 0;
            if (tid == 128) MSK_TRD(3, tri, 8);
          }
        }
        if (tid == 128 && unit_i == 0) MSK_TR(TR_FIRST_EPI_DONE);
      }
      if (!ok) break;
    }
    }
