// Exercises the C++ mirror of the KVCache protocol surface on a machine without a device: empty
// caches, metaState, scheme tables, list-level calls and prompt-cache files never launch a kernel.
#include <cstdio>
#include <string>

#include "../mlx-swift-lm_b200/host/KVCache.hpp"

using namespace kvc::host;

#define EXPECT(cond)                                                          \
    do {                                                                      \
        if (!(cond)) {                                                        \
            std::printf("FAILED line %d: %s\n", __LINE__, #cond);             \
            return 1;                                                         \
        }                                                                     \
    } while (0)

int main(int argc, char **argv) {
    const std::string path = argc > 1 ? argv[1] : "/tmp/host_mirror.safetensors";
    CacheArray caches;
    caches.push_back(std::make_unique<KVCacheSimple>());
    caches.push_back(std::make_unique<RotatingKVCache>(32, 4));
    caches.push_back(std::make_unique<QuantizedKVCache>(32, 4));
    caches.push_back(std::make_unique<TurboQuantKVCache>(4, 3, 4, 7));

    EXPECT(caches[0]->offset() == 0 && !caches[0]->maxSize());
    EXPECT(caches[1]->maxSize() && *caches[1]->maxSize() == 32);
    const auto rot = caches[1]->metaState();
    EXPECT(rot.size() == 6 && rot[0] == "4" && rot[1] == "32" && rot[5] == "modelNative");
    auto *q = dynamic_cast<QuantizedKVCache *>(caches[2].get());
    EXPECT(q && q->groupSize() == 32 && q->bits() == 4);
    EXPECT(caches[0]->isTrimmable() && canTrimPromptCache(caches));
    EXPECT(trimPromptCache(caches, 5) == 0);   // nothing stored yet

    const auto mask = caches[0]->makeMask(1, std::nullopt, false);
    EXPECT(mask.kind == MaskKind::none);
    const auto causal = caches[0]->makeMask(4, std::nullopt, false);
    EXPECT(causal.kind == MaskKind::causal);

    EXPECT(resolveTurboScheme("turbo4v2") == std::make_pair(4, 2));
    EXPECT(resolveTurboScheme("turbo0v4") == std::make_pair(0, 4));
    EXPECT(!resolveTurboScheme("turbo9"));
    EXPECT(resolveAffineScheme("affine4") == std::make_pair(4, 64));

    // below the start threshold nothing converts and the walk is incomplete
    EXPECT(!maybeAffineQuantizeKVCache(caches, 4, 64, 100));
    EXPECT(dynamic_cast<KVCacheSimple *>(caches[0].get()) != nullptr);

    savePromptCache(path, caches, {{"model", "tiny"}, {"note", "two\nlines"}});
    auto [loaded, meta] = loadPromptCache(path);
    EXPECT(loaded.size() == 4 && meta.size() == 2 && meta["model"] == "tiny" && meta["note"] == "two\nlines");
    EXPECT(dynamic_cast<KVCacheSimple *>(loaded[0].get()) && dynamic_cast<RotatingKVCache *>(loaded[1].get()));
    EXPECT(dynamic_cast<QuantizedKVCache *>(loaded[2].get()) && dynamic_cast<TurboQuantKVCache *>(loaded[3].get()));
    EXPECT(loaded[1]->metaState() == caches[1]->metaState());
    EXPECT(loaded[3]->metaState() == caches[3]->metaState());

    // the other classes of the protocol: ChunkedKVCache, CacheList (a composite entry of the layer array)
    {
        ChunkedKVCache chunked(128);
        EXPECT(chunked.startPosition() == 0 && chunked.offset() == 0 && chunked.isTrimmable());
        chunked.prepare({3, 5});
        chunked.finalize();
        const auto cm = chunked.metaState();
        EXPECT(cm.size() == 2 && cm[0] == "128" && cm[1] == "0");
        std::vector<std::unique_ptr<KVCache>> kids;
        kids.push_back(std::make_unique<KVCacheSimple>());
        kids.push_back(std::make_unique<RotatingKVCache>(16, 0));
        CacheArray nested;
        nested.push_back(std::make_unique<CacheList>(std::move(kids)));
        nested.push_back(std::make_unique<ChunkedKVCache>());
        auto *list = dynamic_cast<CacheList *>(nested[0].get());
        EXPECT(list && list->count() == 2 && kvc_kind_of((*list)[1]) == KVC_KIND_ROTATING);
        EXPECT(nested[0]->isTrimmable() && nested[0]->offset() == 0);
        savePromptCache(path, nested, {});
        auto [again, m2] = loadPromptCache(path);
        EXPECT(again.size() == 2 && m2.empty());
        auto *l2 = dynamic_cast<CacheList *>(again[0].get());
        EXPECT(l2 && l2->count() == 2 && kvc_kind_of((*l2)[0]) == KVC_KIND_SIMPLE);
        EXPECT(dynamic_cast<ChunkedKVCache *>(again[1].get()) != nullptr);
        EXPECT(again[0]->metaState() == nested[0]->metaState());
        EXPECT(speculateRewind(again, 5, 2, false) == 0);   // nothing stored: nothing to give back
        const RoPE rope{64, false, 10000.f, 1.f};
        EXPECT(rope.config().dims == 64 && rope.config().traditional == 0);
    }

    bool threw = false;
    try {
        savePromptCache(path, caches, {{"__mlx_lm_state_count", "1"}});
    } catch (const Error &e) {
        threw = e.status == KVC_ERR_INVALID_ARG;
    }
    EXPECT(threw);
    threw = false;
    try {
        (void)loadPromptCache(path + ".missing");
    } catch (const Error &) {
        threw = true;
    }
    EXPECT(threw);
    std::printf("ok\n");
    return 0;
}
