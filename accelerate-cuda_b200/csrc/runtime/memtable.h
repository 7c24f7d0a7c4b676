/*
 * memtable.h -- the device memory table: host-array identity -> device
 * allocation, with pinning, LRU write-back eviction when the device is full,
 * and borrowed ("unmanaged") entries.
 *
 * Replaces Data/Array/Accelerate/CUDA/Array/Remote.hs:91-202 (which wraps the
 * LRU manager of the accelerate package) and the allocation half of
 * Array/Prim.hs:159-186.  Kept from there: allocations are rounded up to 1024
 * bytes and are at least one element (Remote.hs:60-80, Prim.hs:167,186); a
 * failed allocation is not an error but the signal to evict and retry
 * (Remote.hs:63-67); entries in use by device work are pinned and cannot be
 * evicted, and an entry remembers the last asynchronous work that used it
 * (a "waypoint": an event recorded behind that work), which eviction and
 * removal wait for before the memory is written back or freed (withRemote,
 * Remote.hs:113-134); memory registered with
 * insertUnmanaged is never freed by the table (Remote.hs:168-184).
 *
 * The table is header-only and talks to the device through DeviceAllocator,
 * so the eviction logic can be unit-tested on a machine without a GPU by
 * plugging in an allocator with a fixed capacity.
 */
#pragma once
#include <cstddef>
#include <cstdint>
#include <unordered_map>

namespace accb_rt {

struct DeviceAllocator {
    virtual ~DeviceAllocator() {}
    virtual void *alloc(size_t bytes) = 0; /* nullptr when out of memory */
    virtual void release(void *p) = 0;
    virtual bool copy_to_host(void *host, const void *dev, size_t bytes) = 0;
    /* waypoints: opaque tokens that stand for asynchronous work still using an entry */
    virtual void wait_token(void *token) { (void)token; }    /* returns once that work has finished */
    virtual void release_token(void *token) { (void)token; } /* the token is not needed any more */
};

class MemTable {
public:
    struct Entry {
        void *dptr = nullptr;
        size_t bytes = 0;        /* requested size */
        size_t alloc_bytes = 0;  /* rounded size */
        void *host = nullptr;    /* host copy to write back to on eviction (may be null) */
        bool managed = true;     /* false: borrowed from the caller */
        bool resident = true;    /* false: evicted, data lives in `host` */
        int pins = 0;
        uint64_t tick = 0;       /* last use */
        void *waypoint = nullptr; /* token of the last asynchronous work that used the entry, or null */
    };

    static constexpr size_t kGranule = 1024;

    explicit MemTable(DeviceAllocator *a) : alloc_(a) {}
    ~MemTable() { clear(); }

    static size_t round_up(size_t bytes) {
        if (bytes == 0) bytes = 1;
        return (bytes + kGranule - 1) / kGranule * kGranule;
    }

    /* Allocate with eviction.  Returns nullptr only if nothing more can be evicted. */
    void *alloc_raw(size_t bytes) {
        const size_t want = round_up(bytes);
        for (;;) {
            void *p = alloc_->alloc(want);
            if (p) return p;
            if (!evict_one()) return nullptr;
        }
    }

    /* new managed entry; replaces an existing entry with the same key */
    Entry *insert(uint64_t key, size_t bytes, void *host) {
        remove(key);
        void *p = alloc_raw(bytes);
        if (!p) return nullptr;
        Entry e;
        e.dptr = p;
        e.bytes = bytes;
        e.alloc_bytes = round_up(bytes);
        e.host = host;
        e.tick = ++clock_;
        resident_bytes_ += e.alloc_bytes;
        return &(map_[key] = e);
    }

    Entry *insert_unmanaged(uint64_t key, void *dptr, size_t bytes) {
        remove(key);
        Entry e;
        e.dptr = dptr;
        e.bytes = bytes;
        e.alloc_bytes = 0;
        e.managed = false;
        e.tick = ++clock_;
        return &(map_[key] = e);
    }

    /* nullptr if unknown.  Touches the entry. */
    Entry *find(uint64_t key) {
        auto it = map_.find(key);
        if (it == map_.end()) return nullptr;
        it->second.tick = ++clock_;
        return &it->second;
    }

    /* look without touching (does not count as a use) */
    const Entry *peek(uint64_t key) const {
        auto it = map_.find(key);
        return it == map_.end() ? nullptr : &it->second;
    }

    /* Bring an evicted entry back; *needs_upload tells the caller to copy
     * `host` to the device again. */
    Entry *ensure_resident(uint64_t key, bool *needs_upload) {
        *needs_upload = false;
        Entry *e = find(key);
        if (!e || e->resident) return e;
        e->pins++; /* do not pick ourselves as a victim */
        void *p = alloc_raw(e->bytes);
        e->pins--;
        if (!p) return nullptr;
        e->dptr = p;
        e->resident = true;
        resident_bytes_ += e->alloc_bytes;
        *needs_upload = true;
        return e;
    }

    bool pin(uint64_t key) {
        Entry *e = find(key);
        if (!e || !e->resident) return false;
        e->pins++;
        return true;
    }
    bool unpin(uint64_t key) {
        auto it = map_.find(key);
        if (it == map_.end() || it->second.pins <= 0) return false;
        it->second.pins--;
        return true;
    }

    /* The entry was handed to asynchronous work that `token` stands for: the table takes the token over and waits
     * for it before it writes the entry back, frees it or forgets it.  A newer token replaces an older one (work
     * on one stream is ordered; callers that use several streams pass the token of a join). */
    bool set_waypoint(uint64_t key, void *token) {
        auto it = map_.find(key);
        if (it == map_.end()) {
            alloc_->release_token(token);
            return false;
        }
        if (it->second.waypoint) alloc_->release_token(it->second.waypoint);
        it->second.waypoint = token;
        return true;
    }

    bool remove(uint64_t key) {
        auto it = map_.find(key);
        if (it == map_.end()) return false;
        drop(it->second);
        map_.erase(it);
        return true;
    }

    /* free every unpinned managed entry that has a host copy (write-back) or
     * no pins at all when `all` is set */
    size_t reclaim() {
        size_t n = 0;
        while (evict_one()) ++n;
        return n;
    }

    void clear() {
        for (auto &kv : map_) drop(kv.second);
        map_.clear();
    }

    size_t entries() const { return map_.size(); }
    size_t resident_bytes() const { return resident_bytes_; }
    size_t evictions() const { return evictions_; }

private:
    void settle(Entry &e) { /* no asynchronous work uses the entry after this */
        if (!e.waypoint) return;
        alloc_->wait_token(e.waypoint);
        alloc_->release_token(e.waypoint);
        e.waypoint = nullptr;
    }

    void drop(Entry &e) {
        settle(e);
        if (e.managed && e.resident && e.dptr) {
            alloc_->release(e.dptr);
            resident_bytes_ -= e.alloc_bytes;
        }
        e.dptr = nullptr;
    }

    /* write back and free the least recently used evictable entry */
    bool evict_one() {
        Entry *victim = nullptr;
        for (auto &kv : map_) {
            Entry &e = kv.second;
            if (!e.managed || !e.resident || e.pins > 0 || !e.host) continue;
            if (!victim || e.tick < victim->tick) victim = &e;
        }
        if (!victim) return false;
        settle(*victim); /* work enqueued earlier may still read or write it (Remote.hs:127-134) */
        if (!alloc_->copy_to_host(victim->host, victim->dptr, victim->bytes)) return false;
        alloc_->release(victim->dptr);
        resident_bytes_ -= victim->alloc_bytes;
        victim->dptr = nullptr;
        victim->resident = false;
        ++evictions_;
        return true;
    }

    DeviceAllocator *alloc_;
    std::unordered_map<uint64_t, Entry> map_;
    uint64_t clock_ = 0;
    size_t resident_bytes_ = 0;
    size_t evictions_ = 0;
};

}  // namespace accb_rt
