// CPU harness for the device memory table (accelerate-cuda_b200/csrc/runtime/memtable.h):
// the table's eviction / pinning / unmanaged logic driven through a fake device allocator with
// a fixed capacity.  Prints "OK" and exits 0 when every check holds.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <vector>

#include "memtable.h"

using namespace accb_rt;

struct FakeDevice : DeviceAllocator {
    size_t capacity, used = 0;
    std::map<void *, size_t> live;
    int releases = 0, writebacks = 0;
    explicit FakeDevice(size_t cap) : capacity(cap) {}
    void *alloc(size_t bytes) override {
        if (used + bytes > capacity) return nullptr;  // the signal to evict, as cuMemAlloc's OutOfMemory is
        void *p = malloc(bytes);
        live[p] = bytes;
        used += bytes;
        return p;
    }
    void release(void *p) override {
        used -= live.at(p);
        live.erase(p);
        free(p);
        ++releases;
    }
    bool copy_to_host(void *host, const void *dev, size_t bytes) override {
        memcpy(host, dev, bytes);
        ++writebacks;
        log.push_back('c');
        return true;
    }
    // waypoints: a token is a pointer to an int that counts how often it was waited for
    std::vector<char> log;  // 'w' wait, 'r' token released, 'c' copy to host
    void wait_token(void *token) override {
        ++*static_cast<int *>(token);
        log.push_back('w');
    }
    void release_token(void *) override { log.push_back('r'); }
};

#define CHECK(c)                                                        \
    do {                                                                \
        if (!(c)) {                                                     \
            printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #c);      \
            return 1;                                                   \
        }                                                               \
    } while (0)

int main() {
    FakeDevice dev(10 * 1024);
    {
        MemTable t(&dev);
        std::vector<std::vector<char>> host(5, std::vector<char>(3000));
        // sizes are rounded up to 1024-byte granules (Remote.hs:60-80)
        CHECK(MemTable::round_up(1) == 1024 && MemTable::round_up(0) == 1024 && MemTable::round_up(3000) == 3072);
        for (int i = 0; i < 3; ++i) {
            MemTable::Entry *e = t.insert(i, 3000, host[i].data());
            CHECK(e && e->resident);
            memset(e->dptr, 'a' + i, 3000);
        }
        CHECK(t.resident_bytes() == 3 * 3072 && t.evictions() == 0);
        // touching 0 makes 1 the least recently used
        CHECK(t.find(0));
        // a fourth array does not fit: the LRU entry is written back to its host copy and evicted
        MemTable::Entry *e3 = t.insert(3, 3000, host[3].data());
        CHECK(e3 && t.evictions() == 1 && dev.writebacks == 1);
        CHECK(!t.peek(1)->resident && host[1][0] == 'b' && host[1][2999] == 'b');
        CHECK(t.peek(0)->resident && t.peek(2)->resident);
        // bringing 1 back evicts the next LRU entry (2) and asks for a re-upload
        bool upload = false;
        MemTable::Entry *e1 = t.ensure_resident(1, &upload);
        CHECK(e1 && e1->resident && upload && t.evictions() == 2 && !t.peek(2)->resident);
        // pinned entries are never victims (withRemote, Remote.hs:113-134)
        CHECK(t.pin(0) && t.pin(3) && t.pin(1));
        CHECK(t.insert(4, 3000, host[4].data()) == nullptr);  // nothing evictable: allocation fails
        CHECK(t.unpin(0));
        CHECK(t.insert(4, 3000, host[4].data()) != nullptr);  // now 0 can go
        CHECK(!t.peek(0)->resident);
        // entries without a host copy (intermediates) cannot be evicted
        CHECK(t.unpin(3) && t.unpin(1));
        CHECK(t.remove(3) && t.remove(1) && t.remove(4));
        MemTable::Entry *tmp = t.insert(10, 9000, nullptr);
        CHECK(tmp && tmp->resident);
        CHECK(t.insert(11, 3000, nullptr) == nullptr && t.peek(10)->resident);
        // borrowed memory is tracked but never freed by the table (insertUnmanaged, Remote.hs:168-184)
        char borrowed[64];
        int before = dev.releases;
        CHECK(t.insert_unmanaged(20, borrowed, sizeof borrowed));
        CHECK(t.remove(20) && dev.releases == before);
        // reclaim evicts everything evictable (performGC)
        CHECK(t.remove(10));
        CHECK(t.insert(30, 2000, host[0].data()) && t.insert(31, 2000, host[1].data()));
        CHECK(t.reclaim() == 2 && t.resident_bytes() == 0);
        // an entry still used by asynchronous work carries a waypoint: eviction waits for it BEFORE the
        // write-back (Remote.hs:127-134); a newer waypoint replaces the older one; removal waits as well
        CHECK(t.remove(30) && t.remove(31));
        int waits_a = 0, waits_b = 0, waits_c = 0;
        CHECK(t.insert(40, 2000, host[0].data()) && t.insert(41, 2000, host[1].data()));
        CHECK(t.set_waypoint(40, &waits_a));
        CHECK(t.set_waypoint(40, &waits_b));  // releases token a unwaited
        dev.log.clear();
        CHECK(t.find(41));                    // 40 is the LRU entry
        CHECK(t.insert(42, 8000, nullptr));   // needs 40's memory
        CHECK(waits_a == 0 && waits_b == 1 && !t.peek(40)->resident);
        CHECK(dev.log.size() >= 3 && dev.log[0] == 'w' && dev.log[1] == 'r' && dev.log[2] == 'c');
        CHECK(t.set_waypoint(41, &waits_c) && t.remove(41) && waits_c == 1);
        CHECK(!t.set_waypoint(99, &waits_c));  // unknown key: the token is handed back
        CHECK(t.remove(42) && t.remove(40));
    }
    CHECK(dev.used == 0 && dev.live.empty());  // the destructor released what was left
    printf("OK\n");
    return 0;
}
