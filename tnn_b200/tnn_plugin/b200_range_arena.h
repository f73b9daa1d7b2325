// Sub-allocation of blocks from slabs: the host-side logic of the device memory arena, free of any CUDA call so that
// it can be exercised without a GPU.  A slab is one allocation of the backing store (cudaMalloc in the device, a fake
// address range in the self-test); blocks are cut from the smallest free range that fits (best fit over all slabs of the
// arena) and freed ranges merge with their neighbours.  Not thread-safe: the owner serialises calls.
#ifndef TNN_B200_RANGE_ARENA_H_
#define TNN_B200_RANGE_ARENA_H_

#include <cstddef>
#include <cstdint>
#include <functional>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>

namespace tnn_b200 {

class RangeArena {
public:
    using SlabAlloc = std::function<void*(size_t bytes)>;   // returns nullptr on failure
    using SlabFree  = std::function<void(void* base)>;

    struct TakeResult {
        void* ptr         = nullptr;
        size_t length     = 0;   // the block's length after rounding
        size_t new_slab   = 0;   // bytes of the slab this call had to allocate (0: served from a cached slab)
    };
    struct GiveResult {
        bool found        = false;
        size_t length     = 0;
        size_t freed_slab = 0;   // bytes of the slab this call returned to the backing store (unpooled mode only)
    };

    // pooled = false: every block is its own slab, returned to the backing store when freed (the reference's behaviour).
    RangeArena(size_t slab_bytes, size_t align, bool pooled) : slab_bytes_(slab_bytes), align_(align), pooled_(pooled) {}
    ~RangeArena() {
        for (Slab* s : slabs_) delete s;
    }
    RangeArena(const RangeArena&) = delete;
    RangeArena& operator=(const RangeArena&) = delete;

    TakeResult Take(size_t bytes, const SlabAlloc& alloc) {
        TakeResult r;
        const size_t rounded = (bytes ? bytes + align_ - 1 : align_) / align_ * align_;
        Slab* best_slab = nullptr;
        std::map<size_t, size_t>::iterator best_it;
        if (pooled_) {
            size_t best_len = ~static_cast<size_t>(0);
            for (Slab* s : slabs_) {
                for (auto it = s->free_ranges.begin(); it != s->free_ranges.end(); ++it) {
                    if (it->second >= rounded && it->second < best_len) {
                        best_len  = it->second;
                        best_slab = s;
                        best_it   = it;
                    }
                }
            }
        }
        if (!best_slab) {
            // a request above half a slab gets a slab of its own size: it would leave a fragment nobody fits otherwise
            const size_t size = pooled_ ? (rounded > slab_bytes_ / 2 ? rounded : slab_bytes_) : rounded;
            void* base = alloc(size);
            if (!base) return r;
            Slab* s = new Slab();
            s->base   = static_cast<char*>(base);
            s->size   = size;
            s->in_use = 0;
            s->free_ranges[0] = size;
            slabs_.push_back(s);
            best_slab  = s;
            best_it    = s->free_ranges.begin();
            r.new_slab = size;
        }
        const size_t off = best_it->first, len = best_it->second;
        best_slab->free_ranges.erase(best_it);
        if (len > rounded) best_slab->free_ranges[off + rounded] = len - rounded;
        best_slab->in_use += rounded;
        r.ptr    = best_slab->base + off;
        r.length = rounded;
        live_[r.ptr] = Live{best_slab, rounded};
        return r;
    }

    GiveResult Give(void* ptr, const SlabFree& free_slab) {
        GiveResult r;
        auto it = live_.find(ptr);
        if (it == live_.end()) return r;
        const Live l = it->second;
        live_.erase(it);
        r.found  = true;
        r.length = l.length;
        Slab* s  = l.slab;
        size_t off = static_cast<size_t>(static_cast<char*>(ptr) - s->base), len = l.length;
        s->in_use -= len;
        auto next = s->free_ranges.lower_bound(off);
        if (next != s->free_ranges.end() && off + len == next->first) {
            len += next->second;
            next = s->free_ranges.erase(next);
        }
        bool merged = false;
        if (next != s->free_ranges.begin()) {
            auto prev = std::prev(next);
            if (prev->first + prev->second == off) {
                prev->second += len;
                merged = true;
            }
        }
        if (!merged) s->free_ranges[off] = len;
        if (!pooled_ && s->in_use == 0) {
            r.freed_slab = s->size;
            Drop(s, free_slab);
        }
        return r;
    }

    bool Owns(void* ptr) const { return live_.count(ptr) > 0; }

    // Returns every slab without a live block to the backing store; the number of bytes released.
    size_t ReleaseEmpty(const SlabFree& free_slab, size_t* slabs_released = nullptr) {
        size_t released = 0, n = 0;
        for (size_t i = 0; i < slabs_.size();) {
            if (slabs_[i]->in_use == 0) {
                released += slabs_[i]->size;
                ++n;
                Drop(slabs_[i], free_slab);
            } else {
                ++i;
            }
        }
        if (slabs_released) *slabs_released = n;
        return released;
    }

    size_t live_blocks() const { return live_.size(); }
    size_t slab_count() const { return slabs_.size(); }
    size_t bytes_reserved() const {
        size_t n = 0;
        for (const Slab* s : slabs_) n += s->size;
        return n;
    }
    size_t bytes_in_use() const {
        size_t n = 0;
        for (const Slab* s : slabs_) n += s->in_use;
        return n;
    }

    // Structural check for the self-test: live blocks and free ranges tile every slab exactly, free ranges are merged,
    // the per-slab byte counts agree.  Returns an empty string when everything holds.
    std::string CheckInvariants() const {
        std::map<const Slab*, std::map<size_t, size_t>> used;
        for (const auto& kv : live_) {
            const Slab* s = kv.second.slab;
            const size_t off = static_cast<size_t>(static_cast<const char*>(kv.first) - s->base);
            if (off % align_ || kv.second.length % align_) return "a live block is not aligned";
            used[s][off] = kv.second.length;
        }
        for (const Slab* s : slabs_) {
            std::map<size_t, std::pair<size_t, bool>> all;   // offset -> (length, is_free)
            size_t in_use = 0;
            for (const auto& fr : s->free_ranges) {
                if (fr.second == 0) return "an empty free range";
                all[fr.first] = std::make_pair(fr.second, true);
            }
            auto u = used.find(s);
            if (u != used.end()) {
                for (const auto& b : u->second) {
                    if (all.count(b.first)) return "a live block starts where a free range starts";
                    all[b.first] = std::make_pair(b.second, false);
                    in_use += b.second;
                }
            }
            if (in_use != s->in_use) return "a slab's in-use count disagrees with its live blocks";
            size_t at = 0;
            bool prev_free = false;
            for (const auto& e : all) {
                if (e.first != at) return e.first < at ? "two ranges overlap" : "a gap that is neither live nor free";
                if (e.second.second && prev_free) return "two adjacent free ranges were not merged";
                prev_free = e.second.second;
                at += e.second.first;
            }
            if (at != s->size) return "the ranges do not add up to the slab";
        }
        for (const auto& u : used) {
            bool known = false;
            for (const Slab* s : slabs_) known = known || s == u.first;
            if (!known) return "a live block refers to a slab that is gone";
        }
        return std::string();
    }

private:
    struct Slab {
        char* base;
        size_t size;
        size_t in_use;
        std::map<size_t, size_t> free_ranges;   // offset -> length; neighbours merge in O(log n)
    };
    struct Live {
        Slab* slab;
        size_t length;
    };

    void Drop(Slab* s, const SlabFree& free_slab) {
        for (size_t i = 0; i < slabs_.size(); ++i) {
            if (slabs_[i] == s) {
                slabs_.erase(slabs_.begin() + i);
                break;
            }
        }
        free_slab(s->base);
        delete s;
    }

    size_t slab_bytes_, align_;
    bool pooled_;
    std::vector<Slab*> slabs_;
    std::unordered_map<void*, Live> live_;
};

}  // namespace tnn_b200

#endif  // TNN_B200_RANGE_ARENA_H_
