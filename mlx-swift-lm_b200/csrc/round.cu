// Staged speculative rounds (RotatingStagedKVCache.swift:12-130,
// KVCacheRound.swift:87-206, KVCachePlan.swift:219-347), per cache.
//
// A rotating cache cannot take back a multi-token write once the ring has
// wrapped, so during a verify round its new rows are staged beside the ring
// and the model sees logicalView(tail: min(offset, maxSize-1)) ++ staged.
// Commit writes only the accepted prefix through the normal update path and,
// when a plain trim could no longer undo it, keeps a restore point. Append-only
// caches are written through and trimmed back on commit.
#include "cache.h"

#include <algorithm>
#include <memory>

namespace kvc {

namespace {

void copy_view_rows(const kvc_tensor &src, Array4 &dst, int64_t dst_first, cudaStream_t s) {
    if (src.shape[2] == 0) return;
    AppendArgs a;
    a.k_src = src.data; a.v_src = src.data;
    a.ks_sb = src.stride[0]; a.ks_sh = src.stride[1]; a.ks_ss = src.stride[2]; a.ks_sd = src.stride[3];
    a.vs_sb = a.ks_sb; a.vs_sh = a.ks_sh; a.vs_ss = a.ks_ss; a.vs_sd = a.ks_sd;
    a.k_dst = dst.ptr; a.v_dst = dst.ptr;
    a.kd_sb = dst.sb(); a.kd_sh = dst.sh(); a.kd_st = dst.st();
    a.vd_sb = a.kd_sb; a.vd_sh = a.kd_sh; a.vd_st = a.kd_st;
    a.B = (int)src.shape[0]; a.H = (int)src.shape[1]; a.S = (int)src.shape[2];
    a.Dk = (int)src.shape[3]; a.Dv = 0;
    a.pos = dst_first;
    a.esize = (int)dtype_size(src.dtype);
    launch_append(a, s);
}

void snapshot(const Array4 &src, Array4 &dst, int64_t rows, cudaStream_t s) {
    dst.release(s);
    if (!src.allocated()) return;
    dst.alloc(src.B, src.H, std::max<int64_t>(rows, 1), src.W, src.dtype, s);
    copy_view_rows(src.view(rows), dst, 0, s);
}

}  // namespace

void round_begin(kvc_cache *c, int max_positions, kvc_round **out) {
    KVC_REQUIRE(max_positions >= 0, "beginRound: maximumPositions must be non-negative");
    if (c->open_round) fail(KVC_ERR_INVALID_STATE, "a staged round is already open on this cache");
    std::unique_ptr<kvc_round> r(new kvc_round());
    r->cache = c;
    r->max_positions = max_positions;
    r->start_offset = c->offset;
    if (c->cfg.kind == KVC_KIND_ROTATING) {
        r->rotating = true;
        c->open_round = r.get();
    } else {
        // KVCacheRoundStrategyFactory.make (KVCacheRound.swift:183-206): write-through
        // is admitted only if a later trim can undo the whole round.
        if (!cache_is_trimmable_after(c, max_positions))
            fail(KVC_ERR_NOT_TRIMMABLE, "beginRound: the cache could not be rewound after this round");
        r->rotating = false;
    }
    c->restore.valid = false;
    *out = r.release();
}

void round_update(kvc_round *r, const kvc_tensor &k, const kvc_tensor &v, cudaStream_t s,
                  kvc_tensor *ok, kvc_tensor *ov) {
    kvc_cache *c = r->cache;
    if (!r->rotating) {
        cache_update(c, k, v, s, ok, ov);
        return;
    }
    KVC_REQUIRE(k.ndim == 4 && v.ndim == 4, "round update: keys/values must be [B, H, S, D]");
    KVC_REQUIRE(is_float_dtype(k.dtype) && k.dtype == v.dtype, "round update: keys/values must share a floating dtype");
    KVC_REQUIRE(k.shape[0] == v.shape[0] && k.shape[1] == v.shape[1] && k.shape[2] == v.shape[2],
                "round update: keys and values disagree");
    const int64_t S = k.shape[2];
    if (!r->sk.allocated()) {
        const int64_t cap = std::max<int64_t>(std::max<int64_t>(r->max_positions, S), 1);
        r->sk.alloc(k.shape[0], k.shape[1], cap, k.shape[3], k.dtype, s);
        r->sv.alloc(v.shape[0], v.shape[1], cap, v.shape[3], v.dtype, s);
    } else {
        KVC_REQUIRE(k.shape[0] == r->sk.B && k.shape[1] == r->sk.H && k.shape[3] == r->sk.W &&
                        v.shape[3] == r->sv.W && k.dtype == r->sk.dtype,
                    "round update: new rows do not match the staged shape");
        r->sk.ensure(r->staged + S, r->staged, 16, s);
        r->sv.ensure(r->staged + S, r->staged, 16, s);
    }
    copy_view_rows(k, r->sk, r->staged, s);
    copy_view_rows(v, r->sv, r->staged, s);
    r->staged += S;

    // presentation (RotatingStagedKVCache.swift:75-88)
    const int64_t bound = std::min<int64_t>(c->offset, (int64_t)c->cfg.max_size - 1);
    kvc_tensor vk{}, vv{};
    int64_t hist = 0;
    if (bound > 0 && c->k.allocated()) {
        cache_logical_view(c, bound, s, &vk, &vv);
        hist = vk.shape[2];
    }
    if (hist == 0) {
        if (ok) *ok = r->sk.view(r->staged);
        if (ov) *ov = r->sv.view(r->staged);
        return;
    }
    const int64_t total = hist + r->staged;
    auto fit = [&](Array4 &dst, const Array4 &like) {
        if (dst.allocated() && dst.cap >= total && dst.B == like.B && dst.H == like.H && dst.W == like.W &&
            dst.dtype == like.dtype)
            return;
        dst.release(s);
        dst.alloc(like.B, like.H, std::max<int64_t>(total, (int64_t)c->cfg.max_size + r->max_positions), like.W,
                  like.dtype, s);
    };
    fit(r->pk, r->sk);
    fit(r->pv, r->sv);
    copy_view_rows(vk, r->pk, 0, s);
    copy_view_rows(vv, r->pv, 0, s);
    copy_view_rows(r->sk.view(r->staged), r->pk, hist, s);
    copy_view_rows(r->sv.view(r->staged), r->pv, hist, s);
    if (ok) *ok = r->pk.view(total);
    if (ov) *ov = r->pv.view(total);
}

void round_commit(kvc_round *r, int retain, cudaStream_t s) {
    kvc_cache *c = r->cache;
    const int64_t written = r->rotating ? r->staged : c->offset - r->start_offset;
    KVC_REQUIRE(retain >= 0 && retain <= written, "commit: cannot retain more positions than the round wrote");
    if (!r->rotating) {
        // AppendOnlyRoundStrategy.commit (KVCacheRound.swift:101-109)
        if (written > retain) cache_trim(c, written - retain);
        r->closed = true;
        return;
    }
    c->open_round = nullptr;
    r->closed = true;
    // RotatingRoundStrategy.makeRestorePoint (KVCacheRound.swift:133-147): only when a
    // trim could not undo the committed rows.
    RestorePoint rp;
    const bool need_restore = !cache_is_trimmable_after(c, retain) && c->k.allocated();
    if (need_restore) {
        const int64_t rows = c->offset < c->len ? std::max<int64_t>(c->offset, 0) : c->len;
        snapshot(c->k, rp.k, rows, s);
        snapshot(c->v, rp.v, rows, s);
        rp.len = rows;
        rp.offset = c->offset;
        rp.idx = c->idx;
        if (r->staged > 0) {
            snapshot(r->sk, rp.rk, r->staged, s);
            snapshot(r->sv, rp.rv, r->staged, s);
        }
        rp.committed = retain;
        rp.valid = true;
    }
    if (retain > 0 && r->staged > 0) {
        kvc_tensor kt = r->sk.view(retain), vt = r->sv.view(retain);
        cache_update(c, kt, vt, s, nullptr, nullptr);  // clears c->restore
    }
    r->staged = 0;
    if (need_restore) {
        c->restore.k.release(s); c->restore.v.release(s);
        c->restore.rk.release(s); c->restore.rv.release(s);
        c->restore = rp;
    } else {
        c->restore.valid = false;
    }
}

int64_t rewind_last_round(kvc_cache *c, int64_t count, cudaStream_t s) {
    // KVCacheStorage.rewindLastRound (KVCachePlan.swift:305-347), one leaf.
    if (c->open_round) fail(KVC_ERR_INVALID_STATE, "cannot rewind while a staged round is open");
    KVC_REQUIRE(count >= 0, "Rewind count cannot be negative");
    if (count == 0) return 0;
    if (!c->restore.valid) {
        // falls back to the list-level trim, which refuses a non-trimmable cache
        if (!cache_is_trimmable_after(c, 0)) return 0;
        return cache_trim(c, count);
    }
    RestorePoint rp = c->restore;
    c->restore = RestorePoint();
    const int64_t rewound = std::min(count, rp.committed);
    if (rewound <= 0) {
        c->restore = rp;
        return 0;
    }
    // restore state, then metaState (RotatingRestorePoint.restore, KVCacheRound.swift:155-175)
    c->k.release(s); c->v.release(s);
    c->k = rp.k; c->v = rp.v;
    c->len = rp.len; c->offset = rp.offset; c->idx = rp.idx;
    const int64_t replay = rp.committed - rewound;
    if (replay > 0 && rp.rk.allocated()) {
        kvc_tensor kt = rp.rk.view(replay), vt = rp.rv.view(replay);
        cache_update(c, kt, vt, s, nullptr, nullptr);
    }
    rp.rk.release(s); rp.rv.release(s);
    c->restore.valid = false;
    return rewound;
}

}  // namespace kvc
