// Host-side request batching over the paged KV pool: which streams run in the next launch, where their tokens
// live, and the device-side arrays (positions, lengths, page table, cu_seqlens) that the attention entry points
// take.  Header-only, no CUDA: it only fills host vectors.
//
// The reference serves one request at a time: ResidentEngine builds a NativeTalkerEngine whose caches hold
// prefill_rows + generation capacity positions (talker_for_rows, devices/rtx4090-24g/qwen3_tts_1_7b.cu:27206-27222;
// generation_capacity_for, :3112-3128: the next power of two of --max-new-tokens between 256 and 8192) and clears
// the per-request state with reset_request() (:16607).  Here the same guarantee - a request that was admitted can
// always run to its last token - is kept for many requests at once: admission reserves the request's worst case
// in 64-token pages, pages are handed out lazily as the stream grows, and a retired stream's pages go back to the
// free list for the next request.
#pragma once

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <vector>

namespace qm {

constexpr int kBatcherPageTokens = 64;

// generation_capacity_for (17.cu:3112-3128).
inline std::size_t generation_capacity_for(std::size_t requested) {
    if (requested == 0 || requested > 8192) throw std::runtime_error("--max-new-tokens must be in [1,8192]");
    std::size_t capacity = 256;
    while (capacity < requested) capacity <<= 1;
    return capacity;
}

// LIFO free list of page ids 0 .. num_pages-1.
class PageAllocator {
public:
    explicit PageAllocator(int num_pages) {
        if (num_pages < 1) throw std::runtime_error("page pool must hold at least one page");
        free_.reserve((std::size_t)num_pages);
        for (int id = num_pages - 1; id >= 0; --id) free_.push_back(id);
        total_ = num_pages;
    }
    int total() const { return total_; }
    int available() const { return (int)free_.size(); }
    int allocate() {
        if (free_.empty()) throw std::runtime_error("page pool exhausted");
        const int id = free_.back();
        free_.pop_back();
        return id;
    }
    void release(int id) {
        if (id < 0 || id >= total_) throw std::runtime_error("released page id out of range");
        free_.push_back(id);
    }

private:
    std::vector<int> free_;
    int total_ = 0;
};

// One decode launch: row r of every array belongs to slot slots[r].
struct DecodePlan {
    int batch = 0;
    int max_pages = 0;
    std::vector<int32_t> slots;
    std::vector<int64_t> request_ids;
    std::vector<int32_t> positions;     // position of the token appended in this step
    std::vector<int32_t> seq_lens;      // keys attended, the new token included
    std::vector<int32_t> page_table;    // [batch][max_pages], unused entries 0
};

// One packed varlen prefill launch.
struct PrefillPlan {
    int batch = 0;
    int max_pages = 0;
    int total_tokens = 0;
    int max_seqlen = 0;
    std::vector<int32_t> slots;
    std::vector<int32_t> cu_seqlens;    // [batch + 1]
    std::vector<int32_t> page_table;    // [batch][max_pages], unused entries 0
};

class StreamBatcher {
public:
    StreamBatcher(int num_pages, int max_streams, int max_pages_per_stream)
        : allocator_(num_pages), max_pages_(max_pages_per_stream), streams_((std::size_t)max_streams) {
        if (max_streams < 1 || max_pages_per_stream < 1) throw std::runtime_error("invalid batcher geometry");
    }

    int max_pages_per_stream() const { return max_pages_; }
    int free_pages() const { return allocator_.available(); }
    // Pages promised to admitted streams and not yet handed out.
    int reserved_pages() const { return reserved_; }
    int active_streams() const {
        int n = 0;
        for (const Stream& s : streams_) n += s.state != kFree;
        return n;
    }
    int length(int slot) const { return at(slot).length; }
    int generated(int slot) const { return at(slot).generated; }
    bool finished(int slot) const { return at(slot).generated >= at(slot).max_new_tokens; }
    const std::vector<int>& pages(int slot) const { return at(slot).pages; }

    // Admits a request: a slot index, or -1 when no slot is free, the request can never fit one stream's page
    // table, or the pool cannot promise its worst case (prompt + capacity class) next to what is already promised;
    // the caller keeps it queued and tries again after a retire().
    int admit(int64_t request_id, int prompt_tokens, int max_new_tokens) {
        if (prompt_tokens < 1) throw std::runtime_error("resident prefill rows must be positive");
        const int worst_tokens = prompt_tokens + (int)generation_capacity_for((std::size_t)max_new_tokens);
        const int worst_pages = pages_for(worst_tokens);
        if (worst_pages > max_pages_) return -1;
        if (worst_pages > allocator_.available() - reserved_) return -1;
        for (std::size_t slot = 0; slot < streams_.size(); ++slot) {
            Stream& s = streams_[slot];
            if (s.state != kFree) continue;
            s = Stream{};
            s.state = kAdmitted;
            s.request_id = request_id;
            s.prompt_tokens = prompt_tokens;
            s.max_new_tokens = max_new_tokens;
            s.promised = worst_pages;
            reserved_ += worst_pages;
            return (int)slot;
        }
        return -1;
    }

    // Packs the prompts of `slots` (admitted, not yet prefilled) into one varlen launch and hands out their pages.
    PrefillPlan plan_prefill(const std::vector<int>& slots) {
        PrefillPlan plan;
        plan.batch = (int)slots.size();
        plan.max_pages = max_pages_;
        plan.slots.assign(slots.begin(), slots.end());
        plan.cu_seqlens.assign(1, 0);
        plan.page_table.assign((std::size_t)plan.batch * max_pages_, 0);
        for (int row = 0; row < plan.batch; ++row) {
            Stream& s = at(slots[(std::size_t)row]);
            if (s.state != kAdmitted) throw std::runtime_error("prefill of a stream that is not waiting for one");
            grow_to(s, s.prompt_tokens);
            for (std::size_t p = 0; p < s.pages.size(); ++p) plan.page_table[(std::size_t)row * max_pages_ + p] = s.pages[p];
            plan.cu_seqlens.push_back(plan.cu_seqlens.back() + s.prompt_tokens);
            plan.max_seqlen = s.prompt_tokens > plan.max_seqlen ? s.prompt_tokens : plan.max_seqlen;
        }
        plan.total_tokens = plan.cu_seqlens.back();
        return plan;
    }

    // After the prefill launch was issued: the prompts are in the cache.
    void commit_prefill(const PrefillPlan& plan) {
        for (int slot : plan.slots) {
            Stream& s = at(slot);
            s.length = s.prompt_tokens;
            s.state = kRunning;
        }
    }

    // Every running, unfinished stream takes part in the next decode step, in slot order.
    DecodePlan plan_decode_step() {
        DecodePlan plan;
        plan.max_pages = max_pages_;
        for (std::size_t slot = 0; slot < streams_.size(); ++slot) {
            Stream& s = streams_[slot];
            if (s.state != kRunning || s.generated >= s.max_new_tokens) continue;
            grow_to(s, s.length + 1);
            plan.slots.push_back((int32_t)slot);
            plan.request_ids.push_back(s.request_id);
            plan.positions.push_back(s.length);
            plan.seq_lens.push_back(s.length + 1);
        }
        plan.batch = (int)plan.slots.size();
        plan.page_table.assign((std::size_t)plan.batch * max_pages_, 0);
        for (int row = 0; row < plan.batch; ++row) {
            const Stream& s = streams_[(std::size_t)plan.slots[(std::size_t)row]];
            for (std::size_t p = 0; p < s.pages.size(); ++p) plan.page_table[(std::size_t)row * max_pages_ + p] = s.pages[p];
        }
        return plan;
    }

    // After the decode launches of the step were issued.
    void commit_decode_step(const DecodePlan& plan) {
        for (int slot : plan.slots) {
            Stream& s = at(slot);
            s.length += 1;
            s.generated += 1;
        }
    }

    // The request ended (EOS, token limit, cancelled): its pages and what was still promised go back.
    void retire(int slot) {
        Stream& s = at(slot);
        if (s.state == kFree) throw std::runtime_error("retire of a free slot");
        for (int id : s.pages) allocator_.release(id);
        reserved_ -= s.promised - (int)s.pages.size();
        s = Stream{};
    }

private:
    enum State { kFree = 0, kAdmitted = 1, kRunning = 2 };
    struct Stream {
        State state = kFree;
        int64_t request_id = 0;
        int prompt_tokens = 0;
        int max_new_tokens = 0;
        int length = 0;        // tokens in the cache
        int generated = 0;
        int promised = 0;      // pages reserved at admission (handed out or not)
        std::vector<int> pages;
    };

    static int pages_for(int tokens) { return (tokens + kBatcherPageTokens - 1) / kBatcherPageTokens; }
    Stream& at(int slot) {
        if (slot < 0 || (std::size_t)slot >= streams_.size()) throw std::runtime_error("slot out of range");
        return streams_[(std::size_t)slot];
    }
    const Stream& at(int slot) const {
        if (slot < 0 || (std::size_t)slot >= streams_.size()) throw std::runtime_error("slot out of range");
        return streams_[(std::size_t)slot];
    }
    // Hands out pages until `tokens` positions fit; never beyond what admission promised.
    void grow_to(Stream& s, int tokens) {
        const int needed = pages_for(tokens);
        if (needed > s.promised) throw std::runtime_error("stream grew past its generation capacity");
        while ((int)s.pages.size() < needed) {
            s.pages.push_back(allocator_.allocate());
            reserved_ -= 1;
        }
    }

    PageAllocator allocator_;
    int max_pages_ = 0;
    int reserved_ = 0;
    std::vector<Stream> streams_;
};

}  // namespace qm
