// When to start the all-reduce of each gradient bucket during the backward sweep.
//
// The parameter gradients live in one slab, cut into buckets of consecutive parameters.  A bucket's reduction may
// start as soon as every tape op that adds into one of its parameters has run its backward arm; the schedule counts
// those ops down and calls `fire(begin, count)` (floats of the slab) at that moment, and `finish()` fires whatever is
// left, in slab order.  The reduction itself is behind a callback, so the bookkeeping is testable on the CPU with any
// stand-in for the collective (threads, a fake that fails, a rank that is late).
#pragma once
#include <stddef.h>

#include <functional>
#include <vector>

namespace znn {
namespace host {

class BucketSchedule {
public:
    using Fire = std::function<int(size_t begin, size_t count)>;   // returns 0 or an error code

    // offsets[i]: first float of parameter i in the slab (ascending); total: slab length; uses[i]: tape ops that read
    // parameter i (its gradient is complete when all of them have run backward; 0 = never touched this step)
    BucketSchedule(const std::vector<size_t>& offsets, size_t total, size_t bucket_floats, const std::vector<int>& uses,
                   Fire fire)
        : remaining_(uses), fire_(std::move(fire))
    {
        const size_t n = offsets.size();
        bucket_of_.assign(n, 0);
        size_t begin = 0;
        for (size_t i = 0; i < n; i++) {
            const size_t end = (i + 1 < n) ? offsets[i + 1] : total;
            bucket_of_[i] = (int)buckets_.size();
            if (end - begin >= bucket_floats || i + 1 == n) {
                buckets_.push_back(Bucket{begin, end, 0, false});
                begin = end;
            }
        }
        for (size_t i = 0; i < n; i++)
            if (remaining_[i] > 0) buckets_[bucket_of_[i]].pending++;
    }

    // one tape op that reads parameter `param` has run its backward arm
    int after(int param)
    {
        if (error_) return error_;
        if (param < 0 || (size_t)param >= remaining_.size() || remaining_[param] <= 0) return 0;
        if (--remaining_[param] == 0) {
            Bucket& b = buckets_[bucket_of_[param]];
            if (--b.pending == 0) return fire_bucket(b);
        }
        return 0;
    }

    // end of the sweep: buckets that never became complete (parameters without gradient this step) go now
    int finish()
    {
        for (Bucket& b : buckets_) {
            if (error_) return error_;
            if (!b.fired) fire_bucket(b);
        }
        return error_;
    }

    size_t buckets() const { return buckets_.size(); }
    int error() const { return error_; }

private:
    struct Bucket {
        size_t begin, end;
        int pending;
        bool fired;
    };
    int fire_bucket(Bucket& b)
    {
        b.fired = true;
        const int rc = fire_(b.begin, b.end - b.begin);
        if (rc != 0 && error_ == 0) error_ = rc;   // the first failure stops all further reductions of this step
        return rc;
    }
    std::vector<int> remaining_, bucket_of_;
    std::vector<Bucket> buckets_;
    Fire fire_;
    int error_ = 0;
};

}  // namespace host
}  // namespace znn
