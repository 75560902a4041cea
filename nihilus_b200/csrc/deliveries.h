// Host-side bookkeeping of the fused all-gather: which launch has to wait for which announcement of the peers.
// Plain C++ (no CUDA): the same code decides for the library (api.cu: plan_peer_wait) and for the host-only planner that
// the CPU tests drive (nhb_wait_planner_*), which replays whole programs against a model of ranks that run at
// different speeds.
//
// Every rank enqueues the same sequence of delivering launches, so "delivering launch number n" names the same launch
// everywhere, and a rank's announcement counter reaching n means: its rows of launches 1..n have landed on every rank,
// and everything it enqueued before its launch n has run.
#pragma once
#include <algorithm>
#include <cstdint>
#include <vector>

struct nhb_span {
	const char* b = nullptr;
	const char* e = nullptr;
	unsigned long long seq = 0;
};

struct nhb_deliveries {
	unsigned long long seq = 0;// delivering launches enqueued so far
	std::vector<nhb_span> pending;// rows the peers deliver with launch `seq`: whole here once every peer has announced `seq`
	std::vector<nhb_span> reads;// symmetric rows read (or written without delivery) by a launch enqueued before delivering launch `seq`: the peers may deliver into them once they have announced `seq`
};

namespace nhb {

	inline bool spans_overlap(const nhb_span& a, const nhb_span& b) {
		return a.b < b.e && b.b < a.e;
	}
	inline void note_span(std::vector<nhb_span>& v, const nhb_span& s) {
		for (nhb_span& o: v)
			if (o.b == s.b && o.e == s.e) {
				o.seq = std::max(o.seq, s.seq);
				return;
			}
		if (v.size() >= 4096)
			v.erase(v.begin());// the oldest entry: long confirmed by the window unless nothing has been delivered since
		v.push_back(s);
	}
	inline void drop_confirmed(std::vector<nhb_span>& v, unsigned long long target) {
		v.erase(std::remove_if(v.begin(), v.end(), [target](const nhb_span& s) { return s.seq <= target; }), v.end());
	}
	inline bool in_any(const nhb_span* regions, int n_regions, const nhb_span& s) {
		for (int i = 0; i < n_regions; ++i)
			if (spans_overlap(regions[i], s))
				return true;
		return false;
	}

	struct wait_plan {
		bool wait = false;// the launch polls the peers' announcements in its prologue ...
		int lag	  = 0;// ... until each has reached (this rank's completed delivering launches - lag)
	};

	// A launch waits for the peers only as far as it must:
	//   - it reads rows a fused launch delivers: until every peer has announced that launch;
	//   - it writes rows the peers are still delivering into: until every peer has announced that launch;
	//   - it delivers into rows an earlier launch of this context read, or wrote without delivering: until every peer has
	//     announced the first delivering launch enqueued at or after that launch (the peers' copies of those rows are then no
	//     longer in use).  If there is no such launch yet, the best it can ask for is the latest one;
	//   - every second delivering launch: until every peer is within `window` delivering launches of this rank, which
	//     bounds how far ranks drift apart (window + 1) and with it what readers this library does not know of (other
	//     kernels on the stream) may assume.  window = 0: every launch waits for every earlier delivery.
	// Everything else proceeds while the exchange is still in flight.  What the wait confirms is forgotten.
	// regions: the symmetric allocations (only rows inside them can be delivered); in / out: what the launch reads and
	// writes; `delivers`: the rows in `out` are completed on every rank.
	inline wait_plan plan_wait(nhb_deliveries& d, int window_opt, const nhb_span* regions, int n_regions, const nhb_span* in, int n_in, const nhb_span* out,
		int n_out, bool delivers) {
		unsigned long long need = 0;
		for (int i = 0; i < n_in; ++i) {
			if (!in_any(regions, n_regions, in[i]))
				continue;
			for (const nhb_span& p: d.pending)
				if (spans_overlap(p, in[i]))
					need = std::max(need, p.seq);
		}
		for (int i = 0; i < n_out; ++i) {
			// rows the peers are still delivering into must have landed before anything is written over them here
			for (const nhb_span& p: d.pending)
				if (spans_overlap(p, out[i]))
					need = std::max(need, p.seq);
			if (delivers)
				for (const nhb_span& r: d.reads)
					if (spans_overlap(r, out[i]))
						need = std::max(need, std::min(r.seq, d.seq));
		}
		const unsigned long long window = static_cast<unsigned long long>(window_opt < 0 ? 0 : window_opt);
		const bool check_window			= window == 0 || (delivers && (d.seq & 1) == 0);
		const unsigned long long target = std::max(need, check_window && d.seq > window ? d.seq - window : 0ull);
		wait_plan plan;
		plan.wait = target != 0;
		plan.lag  = plan.wait ? static_cast<int>(d.seq - target) : 0;
		drop_confirmed(d.pending, target);
		drop_confirmed(d.reads, target);
		for (int i = 0; i < n_in; ++i)
			if (in_any(regions, n_regions, in[i]))
				note_span(d.reads, nhb_span{ in[i].b, in[i].e, d.seq + 1 });
		if (delivers) {
			++d.seq;
			for (int i = 0; i < n_out; ++i)
				note_span(d.pending, nhb_span{ out[i].b, out[i].e, d.seq });
		} else {
			// rows written here without delivery (a weight kept whole on every rank) are, for the peers' later deliveries into
			// them, like rows read here: a peer must not deliver over them before this launch has run
			for (int i = 0; i < n_out; ++i)
				if (in_any(regions, n_regions, out[i]))
					note_span(d.reads, nhb_span{ out[i].b, out[i].e, d.seq + 1 });
		}
		return plan;
	}

	// ---- recorded launch sequences (CUDA graphs) ----
	// The lag of a recorded launch is frozen, and a replay may follow any history.  So a capture begins by assuming that
	// every earlier delivery is unconfirmed and every symmetric row was just read (the first recorded launches then wait for
	// "everything before the graph"), and what one replay leaves behind is kept relative to where the replay starts.
	struct replay_record {
		unsigned long long n_deliver = 0;// delivering launches in the recording
		std::vector<nhb_span> pending, reads;// left unconfirmed at its end, seq relative to its start
	};
	inline nhb_span all_memory(unsigned long long seq) {
		return nhb_span{ reinterpret_cast<const char*>(uintptr_t(1)), reinterpret_cast<const char*>(~uintptr_t(0)), seq };
	}
	inline unsigned long long capture_begin(nhb_deliveries& d) {
		if (d.seq > 0) {
			note_span(d.pending, all_memory(d.seq));
			note_span(d.reads, all_memory(d.seq));
		}
		return d.seq;
	}
	inline replay_record capture_end(const nhb_deliveries& d, unsigned long long seq0) {
		replay_record r;
		r.n_deliver = d.seq - seq0;
		for (const nhb_span& p: d.pending)
			if (p.seq > seq0)
				r.pending.push_back(nhb_span{ p.b, p.e, p.seq - seq0 });
		for (const nhb_span& x: d.reads)
			if (x.seq > seq0)
				r.reads.push_back(nhb_span{ x.b, x.e, x.seq - seq0 });
		return r;
	}
	inline void replayed(nhb_deliveries& d, const replay_record& r) {
		const unsigned long long base = d.seq;
		d.seq += r.n_deliver;
		for (const nhb_span& p: r.pending)
			note_span(d.pending, nhb_span{ p.b, p.e, base + p.seq });
		for (const nhb_span& x: r.reads)
			note_span(d.reads, nhb_span{ x.b, x.e, base + x.seq });
	}

	// a wait for everything delivered so far (nhb_sync, nhb_all_gather*, in front of kernels that do not wait themselves)
	inline bool plan_wait_all(nhb_deliveries& d) {
		if (d.pending.empty())
			return false;
		d.pending.clear();
		drop_confirmed(d.reads, d.seq);
		return true;
	}

}
