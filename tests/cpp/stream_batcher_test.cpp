// CPU-only checks of host/stream_batcher.hpp: a scripted scenario with known answers, the refusal cases, and a
// seeded random simulation that checks the invariants after every action (no page owned twice, free + owned =
// total, promises never exceed what is free, plans describe exactly the running streams).  Exit code 0 = pass.
#include <cstdio>
#include <cstdlib>
#include <iterator>
#include <map>
#include <set>
#include <vector>

#include "stream_batcher.hpp"

#define CHECK(cond)                                                        \
    do {                                                                   \
        if (!(cond)) {                                                     \
            std::printf("line %d: check failed: %s\n", __LINE__, #cond);   \
            return 1;                                                      \
        }                                                                  \
    } while (0)

static uint64_t next_u64(uint64_t& state) {      // SplitMix64
    state += 0x9e3779b97f4a7c15ull;
    uint64_t z = state;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

static int scripted() {
    CHECK(qm::generation_capacity_for(1) == 256);
    CHECK(qm::generation_capacity_for(256) == 256);
    CHECK(qm::generation_capacity_for(257) == 512);
    CHECK(qm::generation_capacity_for(8192) == 8192);
    bool threw = false;
    try { qm::generation_capacity_for(8193); } catch (const std::runtime_error&) { threw = true; }
    CHECK(threw);

    // 20 pages; a request of 70 prompt tokens and up to 100 new ones is promised ceil((70 + 256) / 64) = 6 pages
    qm::StreamBatcher b(/*num_pages=*/20, /*max_streams=*/3, /*max_pages_per_stream=*/8);
    const int a = b.admit(1001, 70, 100);
    CHECK(a == 0 && b.reserved_pages() == 6 && b.free_pages() == 20);
    const int c = b.admit(1002, 130, 256);          // ceil(386 / 64) = 7
    CHECK(c == 1 && b.reserved_pages() == 13);
    CHECK(b.admit(1003, 200, 300) == -1);           // 712 tokens = 12 pages > 8 per stream
    CHECK(b.admit(1003, 10, 256) == 2);             // 5 pages: 18 promised of 20
    CHECK(b.admit(1004, 10, 10) == -1);             // no slot left
    b.retire(2);
    CHECK(b.reserved_pages() == 13 && b.active_streams() == 2);

    qm::PrefillPlan p = b.plan_prefill({a, c});
    CHECK(p.batch == 2 && p.total_tokens == 200 && p.max_seqlen == 130);
    CHECK(p.cu_seqlens.size() == 3 && p.cu_seqlens[1] == 70 && p.cu_seqlens[2] == 200);
    CHECK(b.pages(a).size() == 2 && b.pages(c).size() == 3);
    CHECK(b.free_pages() == 15 && b.reserved_pages() == 8);
    CHECK(p.page_table[0] == b.pages(a)[0] && p.page_table[1] == b.pages(a)[1] && p.page_table[8 + 2] == b.pages(c)[2]);
    qm::DecodePlan none = b.plan_decode_step();
    CHECK(none.batch == 0);                          // nothing runs before its prefill is committed
    b.commit_prefill(p);
    CHECK(b.length(a) == 70 && b.length(c) == 130);

    qm::DecodePlan d = b.plan_decode_step();
    CHECK(d.batch == 2 && d.positions[0] == 70 && d.seq_lens[0] == 71 && d.positions[1] == 130 && d.seq_lens[1] == 131);
    CHECK(d.request_ids[0] == 1001 && d.request_ids[1] == 1002);
    CHECK(b.pages(a).size() == 2 && b.pages(c).size() == 3);       // positions 70 and 130 lie in pages already held
    b.commit_decode_step(d);
    // stream a crosses into its third page at position 128
    for (int step = 0; step < 57; ++step) { d = b.plan_decode_step(); b.commit_decode_step(d); }
    CHECK(b.length(a) == 128 && b.pages(a).size() == 2);
    d = b.plan_decode_step();
    CHECK(b.pages(a).size() == 3 && d.page_table[2] == b.pages(a)[2]);
    b.commit_decode_step(d);
    // stream a stops after its 100 new tokens and is left out of later plans
    while (!b.finished(a)) { d = b.plan_decode_step(); b.commit_decode_step(d); }
    CHECK(b.generated(a) == 100 && b.length(a) == 170);
    d = b.plan_decode_step();
    CHECK(d.batch == 1 && d.slots[0] == c);
    const std::vector<int> held = b.pages(a);
    b.retire(a);
    CHECK(b.free_pages() + (int)b.pages(c).size() == 20);
    // the freed pages serve the next request
    const int e = b.admit(1005, 64, 1);
    CHECK(e == 0);
    qm::PrefillPlan pe = b.plan_prefill({e});
    CHECK(pe.page_table[0] == held.back());          // LIFO: the page released last comes back first
    return 0;
}

static int randomized(uint64_t seed) {
    const int num_pages = 64, max_streams = 6, max_pages = 12;
    qm::StreamBatcher b(num_pages, max_streams, max_pages);
    std::map<int, int> state;        // slot -> 1 admitted, 2 running
    uint64_t rng = seed;
    int64_t next_id = 1;
    for (int action = 0; action < 4000; ++action) {
        const uint64_t draw = next_u64(rng) % 10;
        if (draw < 2) {
            const int prompt = 1 + (int)(next_u64(rng) % 300);
            const int budget = 1 + (int)(next_u64(rng) % 400);
            const int slot = b.admit(next_id++, prompt, budget);
            if (slot >= 0) { CHECK(state.count(slot) == 0); state[slot] = 1; }
        } else if (draw < 4) {
            std::vector<int> waiting;
            for (auto& kv : state) if (kv.second == 1) waiting.push_back(kv.first);
            if (!waiting.empty()) {
                qm::PrefillPlan p = b.plan_prefill(waiting);
                CHECK(p.batch == (int)waiting.size() && p.cu_seqlens.back() == p.total_tokens);
                b.commit_prefill(p);
                for (int s : waiting) state[s] = 2;
            }
        } else if (draw < 9) {
            qm::DecodePlan d = b.plan_decode_step();
            int expected = 0;
            for (auto& kv : state) expected += kv.second == 2 && !b.finished(kv.first);
            CHECK(d.batch == expected);
            for (int row = 0; row < d.batch; ++row) {
                const int slot = d.slots[(size_t)row];
                CHECK(d.positions[(size_t)row] == b.length(slot) && d.seq_lens[(size_t)row] == b.length(slot) + 1);
                const int page_index = d.positions[(size_t)row] / 64;
                CHECK(page_index < (int)b.pages(slot).size());
                CHECK(d.page_table[(size_t)row * max_pages + page_index] == b.pages(slot)[(size_t)page_index]);
            }
            b.commit_decode_step(d);
        } else if (!state.empty()) {
            auto it = state.begin();
            std::advance(it, (long)(next_u64(rng) % state.size()));
            b.retire(it->first);
            state.erase(it);
        }
        // invariants
        std::set<int> owned;
        int owned_count = 0;
        for (auto& kv : state)
            for (int id : b.pages(kv.first)) { CHECK(id >= 0 && id < num_pages); owned.insert(id); ++owned_count; }
        CHECK((int)owned.size() == owned_count);                       // no page owned twice
        CHECK(b.free_pages() + owned_count == num_pages);
        CHECK(b.reserved_pages() >= 0 && b.reserved_pages() <= b.free_pages());
        CHECK(b.active_streams() == (int)state.size());
    }
    return 0;
}

int main() {
    if (int rc = scripted()) return rc;
    for (uint64_t seed = 1; seed <= 5; ++seed)
        if (int rc = randomized(seed)) return rc;
    std::printf("STREAM_BATCHER_OK\n");
    return 0;
}
