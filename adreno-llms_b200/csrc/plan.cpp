// Host side of the resident decode step: which recorded operators may share one launch
// (analyze_run), and the device tables of such a run (build_run).  See plan.h.
#include "plan.h"

#include <cstring>

#include "stream_core.cuh"

namespace nnb {

namespace {

struct Region {
    uintptr_t base;
    size_t bytes;
    int writer;       // operator of the run that wrote it last, -1: still the contents from before the run
    int writer_seg;
    bool is_index;    // the arg-max result word
    int old_updater;  // operator whose in-place epilogue read the contents from before the run (-1: none)
    bool all_inplace; // every writer so far updated the range in place
    std::vector<int> old_readers;  // operators that read, as their x, the contents from before the run
};

bool overlaps(uintptr_t a, size_t an, uintptr_t b, size_t bn) { return a < b + bn && b < a + an; }

}  // namespace

// The rules.  Inside a run nothing orders two operators except the activations themselves: an
// operator starts when the words of its x carry the epoch of the operator that produces them, and an
// in-place epilogue takes each previous value from the word of the operator that wrote it.  So
//   (1) every read must be of a whole output of one earlier operator (or of memory the run has not
//       written so far): the same address range, never a part of one or a range across two;
//   (2) values produced inside the run are read from their published copy, which is private to its
//       producer, and of all writers of a range only the last stores to the range itself: reads and
//       writes of the run's own values can therefore never collide;
//   (3) what can collide is a store to a range with reads of that range's contents from before the
//       run (as some operator's x, or by the first in-place update of the range).  Those reads are
//       ordered before the store when the reader lies on the chain of x producers behind the writer
//       (all of a reader's tiles are done before an operator that consumes its output starts), or
//       row by row when every writer of the range updates it in place, each from the previous
//       writer's published values.
int analyze_run(const std::vector<HazardOp>& ops, int first, std::vector<OpDeps>* deps) {
    deps->clear();
    std::vector<Region> regs;
    int n_argmax = 0;
    const int total = (int)ops.size();
    int i = first;
    for (; i < total && i - first < PLAN_MAX_OPS; ++i) {
        const HazardOp& o = ops[i];
        const int rel = i - first;
        // -- x --
        int x_reg = -1;
        bool ok = true;
        for (size_t r = 0; r < regs.size() && ok; ++r) {
            if (!overlaps(o.x, o.x_bytes, regs[r].base, regs[r].bytes)) continue;
            if (regs[r].base == o.x && regs[r].bytes == o.x_bytes && !regs[r].is_index) x_reg = (int)r;
            else ok = false;  // part of an earlier output, or more than one
        }
        const int x_dep = (ok && x_reg >= 0) ? regs[x_reg].writer : -1;
        // is operator j on the chain of x producers behind this operator?
        auto in_chain = [&](int j) {
            for (int cur = x_dep; cur >= 0; cur = (*deps)[cur].x_dep) {
                if (cur == j) return true;
                if (cur < j) return false;
            }
            return false;
        };
        // -- outputs --
        int out_reg[4] = {-1, -1, -1, -1};
        const int nweights = o.has_argmax ? o.nout - 1 : o.nout;
        for (int k = 0; k < o.nout && ok; ++k) {
            if (overlaps(o.out[k], o.out_bytes[k], o.x, o.x_bytes)) ok = false;  // in place on its own input
            for (int k2 = 0; k2 < k && ok; ++k2)
                if (overlaps(o.out[k], o.out_bytes[k], o.out[k2], o.out_bytes[k2])) ok = false;
            const bool index_word = o.has_argmax && k == nweights;
            for (size_t r = 0; r < regs.size() && ok; ++r) {
                if (!overlaps(o.out[k], o.out_bytes[k], regs[r].base, regs[r].bytes)) continue;
                if (regs[r].base == o.out[k] && regs[r].bytes == o.out_bytes[k] && regs[r].is_index == index_word && !index_word) out_reg[k] = (int)r;
                else ok = false;
            }
            if (!ok || out_reg[k] < 0) continue;
            const Region& R = regs[out_reg[k]];
            for (int j : R.old_readers)
                if (!in_chain(j)) ok = false;
            if (R.old_updater >= 0 && !(o.inplace && k == 0 && R.all_inplace) && !in_chain(R.old_updater)) ok = false;
        }
        if (o.has_argmax && ++n_argmax > 1) ok = false;  // the reduction words of the fused pick are shared
        if (!ok) break;

        // -- accepted: record the dependencies and update the ranges --
        OpDeps d;
        if (x_reg >= 0) {
            Region& R = regs[x_reg];
            if (R.writer >= 0) {
                d.x_dep = R.writer;
                d.x_dep_seg = R.writer_seg;
                (*deps)[R.writer].publish[R.writer_seg] = true;
            } else {
                R.old_readers.push_back(rel);
            }
        } else {
            regs.push_back(Region{o.x, o.x_bytes, -1, 0, false, -1, true, {rel}});
        }
        for (int k = 0; k < o.nout; ++k) {
            const bool index_word = o.has_argmax && k == nweights;
            if (out_reg[k] >= 0) {
                Region& R = regs[out_reg[k]];
                if (R.writer >= 0) {
                    if (o.inplace && k == 0) {
                        d.res_dep = R.writer;
                        d.res_dep_seg = R.writer_seg;
                        (*deps)[R.writer].publish[R.writer_seg] = true;
                    }
                    (*deps)[R.writer].store[R.writer_seg] = false;  // overwritten before the run ends
                } else if (o.inplace && k == 0) {
                    R.old_updater = rel;
                }
                if (!(o.inplace && k == 0)) R.all_inplace = false;
                R.writer = rel;
                R.writer_seg = k;
                R.old_readers.clear();
            } else {
                const bool upd = o.inplace && k == 0;
                regs.push_back(Region{o.out[k], o.out_bytes[k], rel, k, index_word, upd ? rel : -1, upd, {}});
            }
        }
        deps->push_back(d);
    }
    return i - first;
}

void free_run(PlanRun* run) {
    if (run->d_ops) cudaFree(run->d_ops);
    if (run->d_tiles) cudaFree(run->d_tiles);
    if (run->d_ll) cudaFree(run->d_ll);
    if (run->d_bias) cudaFree(run->d_bias);
    if (run->d_state) cudaFree(run->d_state);
    *run = PlanRun();
}

cudaError_t build_run(const std::vector<RecordedOp>& rec, const std::vector<OpDeps>& deps, int first, int count, int sm_count, size_t smem_limit,
                      int* status_dev, PlanRun* run, const char** reason) {
    *run = PlanRun();
    *reason = "";
    run->first = first;
    run->count = count;
    const int G = sm_count;  // one resident block per multiprocessor
    std::vector<PlanOp> ops((size_t)count);
    std::vector<int2> tiles((size_t)count);
    memset(ops.data(), 0, ops.size() * sizeof(PlanOp));
    // published copies: one private array of 8-byte words per output that an operator of the run reads
    std::vector<size_t> ll_off((size_t)count * 3, (size_t)-1);
    size_t ll_words = 0;
    for (int i = 0; i < count; ++i)
        for (int k = 0; k < 3; ++k)
            if (deps[i].publish[k]) {
                ll_off[(size_t)i * 3 + k] = ll_words;
                ll_words += ((size_t)rec[first + i].a.seg[k].N + 1) / 2;
                ll_words = (ll_words + 15) & ~(size_t)15;  // 128-byte lines of their own
            }
    cudaError_t e;
    if (ll_words) {
        if ((e = cudaMalloc((void**)&run->d_ll, ll_words * 8)) != cudaSuccess) return e;
        if ((e = cudaMemset(run->d_ll, 0, ll_words * 8)) != cudaSuccess) return e;
    }
    int k_ll = 0, x_bytes = 0, ctab_bytes = 0, k_norm = 0, max_item = 0;
    long long tile_start = 0;
    std::vector<const uint16_t*> bias((size_t)count * 3, nullptr);
    bool any_bias = false;
    for (int i = 0; i < count; ++i) {
        const RecordedOp& r = rec[first + i];
        const LinArgs& a = r.a;
        const OpDeps& d = deps[i];
        PlanOp& o = ops[i];
        PlanOpScalars& s = o.s;
        const bool dual = a.epi == EPI_SWIGLU;
        const int rowbytes = fmt_row_bytes(r.fmt, a.K);
        const int warp_rows = dual ? 16 : WARP_ROWS;
        const int tile_rows = r.p.kw == 1 ? NCW * warp_rows : warp_rows;
        s.fmt = r.fmt;
        s.epi = a.epi;
        s.dual = dual ? 1 : 0;
        s.ksplit = r.p.kw > 1 ? 1 : 0;
        s.kcb = r.p.kcb;
        s.rowbytes = rowbytes;
        s.nchunks = (rowbytes + r.p.kcb - 1) / r.p.kcb;
        s.groups = s.ksplit ? (s.nchunks + NCW - 1) / NCW : s.nchunks;
        s.K = a.K;
        s.nseg = a.nseg;
        s.item_bytes = stage_bytes_of(r.fmt, r.p.kcb);
        s.nbox = stage_nbox(r.p.kcb);
        size_t wbytes = 0;
        for (int k = 0; k < a.nseg; ++k) wbytes += (size_t)a.seg[k].N * rowbytes;
        s.flags = (wbytes > ((size_t)96 << 20) ? PLAN_EVICT_FIRST : 0) | (r.fmt == FMT_Q4 ? PLAN_SCALE_TMA : 0);
        if (r.fmt == FMT_INT8) {
            // the row scales are static data like the weights: the producer brings them along
            bool aligned = true;
            for (int k = 0; k < a.nseg; ++k) aligned = aligned && (reinterpret_cast<uintptr_t>(a.seg[k].scale) & 15) == 0;
            if (dual) aligned = aligned && (reinterpret_cast<uintptr_t>(a.scale2) & 15) == 0;
            if (aligned) {
                s.flags |= PLAN_ROW_SCALES;
                s.scale_off = s.item_bytes;
                s.item_bytes += PLAN_ROW_SCALE_BYTES;
            }
        }
        int t0 = 0;
        for (int k = 0; k < a.nseg; ++k) {
            PlanSeg& sg = s.seg[k];
            sg.scale = a.seg[k].scale;
            sg.out = d.store[k] ? a.seg[k].out : nullptr;
            sg.ll_out = d.publish[k] ? run->d_ll + ll_off[(size_t)i * 3 + k] : nullptr;
            sg.N = a.seg[k].N;
            sg.tile0 = t0;
            t0 += (a.seg[k].N + tile_rows - 1) / tile_rows;
            if (!make_weight_map(&o.tm[k], a.seg[k].W, a.seg[k].N, rowbytes, tile_rows)) { *reason = "weight view"; return cudaErrorInvalidValue; }
        }
        if (dual && !make_weight_map(&o.tm[3], a.W2, a.seg[0].N, rowbytes, tile_rows)) { *reason = "weight view"; return cudaErrorInvalidValue; }
        if (r.fmt == FMT_Q4) {
            const uint16_t* sbase[4];
            int srow = 0;
            const int bw = r.p.kcb / 8;
            bool ok = q4_scale_views(a, sbase, &srow);
            for (int k = 0; ok && k < a.nseg; ++k) ok = make_scale_map(&o.tm_s[k], sbase[k], a.seg[k].N, srow, bw, tile_rows);
            if (ok && dual) ok = make_scale_map(&o.tm_s[3], sbase[3], a.seg[0].N, srow, bw, tile_rows);
            if (!ok) { *reason = "scale view"; return cudaErrorInvalidValue; }
        }
        for (int k = 0; k < a.nseg; ++k)
            if (a.seg[k].bias) {
                s.flags |= PLAN_BIAS;
                bias[(size_t)i * 3 + k] = a.seg[k].bias;
                any_bias = true;
            }
        s.ntiles = t0;
        s.tile_start = (int)(tile_start % G);
        tiles[i] = make_int2(s.tile_start, s.ntiles);
        tile_start += t0;
        s.nblocks = t0 < G ? t0 : G;
        s.scale2 = a.scale2;
        s.epoch = i + 1;
        if (d.x_dep >= 0) {
            s.x = nullptr;
            s.x_ll = run->d_ll + ll_off[(size_t)d.x_dep * 3 + d.x_dep_seg];
            s.x_epoch = d.x_dep + 1;
            if (a.K > k_ll) k_ll = a.K;
        } else {
            s.x = a.x;
        }
        if (a.epi == EPI_RESIDUAL || a.epi == EPI_SILU_GATE) {
            if (d.res_dep >= 0) {
                s.res_ll = run->d_ll + ll_off[(size_t)d.res_dep * 3 + d.res_dep_seg];
                s.res_epoch = d.res_dep + 1;
            } else {
                s.res = a.seg[0].out;
            }
        }
        s.norm_w = a.norm_w;
        s.norm_eps = a.norm_eps;
        if (a.norm_w && a.K > k_norm) k_norm = a.K;
        s.argmax_slot = a.argmax_slot;
        s.argmax_done = a.argmax_done;
        s.argmax_out = a.argmax_out;
        s.argmax_base = a.argmax_base;
        if (x_bytes_of(r.fmt, 1, a.K) > x_bytes) x_bytes = x_bytes_of(r.fmt, 1, a.K);
        if (ctab_bytes_of(r.fmt, 1, a.K) > ctab_bytes) ctab_bytes = ctab_bytes_of(r.fmt, 1, a.K);
        if (s.item_bytes > max_item) max_item = s.item_bytes;
    }
    // shared-memory layout of the run
    auto up128 = [](int v) { return (v + 127) / 128 * 128; };
    PlanParams& P = run->params;
    P.nops = count;
    P.off_tiles = PLAN_HDR_BYTES;
    P.off_desc = P.off_tiles + up128(count * (int)sizeof(int2));
    P.off_xraw = P.off_desc + 2 * (int)sizeof(PlanOpScalars);
    P.off_xs = P.off_xraw + up128(k_ll * 2);
    P.off_ctab = P.off_xs + x_bytes;
    P.off_norm = P.off_ctab + up128(ctab_bytes);
    P.off_gamma = P.off_norm + up128(k_norm * 2);
    P.off_red = P.off_gamma + up128(k_norm * 2);
    P.off_ring = (P.off_red + red_bytes_of(1) + 1023) / 1024 * 1024;
    const long long room = (long long)smem_limit - P.off_ring - 1024;  // 1 KB of slack to align the ring
    P.ring_bytes = room > 0 ? (int)(room / 1024 * 1024) : 0;
    if (P.ring_bytes < 2 * max_item) { *reason = "activations leave too little shared memory for the weight ring"; return cudaErrorInvalidValue; }
    run->smem = (size_t)P.off_ring + 1024 + (size_t)P.ring_bytes;
    run->grid = G;
    if ((e = cudaMalloc((void**)&run->d_ops, ops.size() * sizeof(PlanOp))) != cudaSuccess) return e;
    if ((e = cudaMemcpy(run->d_ops, ops.data(), ops.size() * sizeof(PlanOp), cudaMemcpyHostToDevice)) != cudaSuccess) return e;
    if ((e = cudaMalloc((void**)&run->d_tiles, tiles.size() * sizeof(int2))) != cudaSuccess) return e;
    if ((e = cudaMemcpy(run->d_tiles, tiles.data(), tiles.size() * sizeof(int2), cudaMemcpyHostToDevice)) != cudaSuccess) return e;
    if ((e = cudaMalloc((void**)&run->d_state, 64)) != cudaSuccess) return e;
    if ((e = cudaMemset(run->d_state, 0, 64)) != cudaSuccess) return e;
    P.ops = run->d_ops;
    P.op_tiles = run->d_tiles;
    P.state = run->d_state;
    P.status = status_dev;
    P.wait_cycles = 400000000ll;  // about 0.2 s of multiprocessor clocks
    P.drop_publish_op = -1;
    P.bias = nullptr;
    if (any_bias) {
        if ((e = cudaMalloc((void**)&run->d_bias, bias.size() * sizeof(const uint16_t*))) != cudaSuccess) return e;
        if ((e = cudaMemcpy(run->d_bias, bias.data(), bias.size() * sizeof(const uint16_t*), cudaMemcpyHostToDevice)) != cudaSuccess) return e;
        P.bias = run->d_bias;
    }
    return cudaSuccess;
}

}  // namespace nnb
