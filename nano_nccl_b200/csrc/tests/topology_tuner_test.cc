// Host-only logic: process topology validation, ring edge resolution, transport plans, the
// tuner's rule table and the NVLink tile geometry.  No GPU needed.
// Mirrors the reference's tests/p2p_topology.cu (plan behaviour) and the edge-resolution rules of
// src/collective/all_reduce/mpi_communicator.cc:235-293.
#include "collective/tuner.h"
#include "kernels/launch.h"
#include "test_util.h"
#include "gemm/gemm.h"
#include "collective/teardown.h"
#include "topology/topology.h"

#include <algorithm>
#include <cstdlib>

using namespace nano_nccl;

static std::vector<RankInfo> ranks(int n, int per_host, bool peer_access) {
    std::vector<RankInfo> v(n);
    for (int r = 0; r < n; ++r) {
        v[r].node_id = 100 + r / per_host;
        v[r].device = r % per_host;
        v[r].uuid[0] = static_cast<unsigned char>(r + 1);
        v[r].can_access_next = peer_access ? 1 : 0;
    }
    return v;
}

int main() {
    {   // teardown policy: release when the drain worked; otherwise quarantine unless fail-stop was asked for
        using nano_nccl::TeardownAction;
        using nano_nccl::decide_teardown;
        CHECK(decide_teardown(false, "") == TeardownAction::Release);
        CHECK(decide_teardown(false, "abort") == TeardownAction::Release);
        CHECK(decide_teardown(true, "") == TeardownAction::Quarantine);
        CHECK(decide_teardown(true, "quarantine") == TeardownAction::Quarantine);
        CHECK(decide_teardown(true, "abort") == TeardownAction::Abort);
        CHECK_THROWS_WITH(decide_teardown(true, "ignore"), "NANO_NCCL_TEARDOWN");
    }
    {   // topology validation
        ProcessTopology t;
        t.global_rank_count = 4;
        t.local_rank_offset = 1;
        t.devices = {0};
        t.edge_kinds.assign(4, TransportKind::P2p);
        validate_topology(t);
        t.devices = {0, 1};
        CHECK_THROWS_WITH(validate_topology(t), "exactly one local GPU");
        t.devices = {0};
        t.edge_kinds[2] = TransportKind::Auto;
        CHECK_THROWS_WITH(validate_topology(t), "unresolved transport");
        t.edge_kinds[2] = TransportKind::Mixed;
        CHECK_THROWS_WITH(validate_topology(t), "unresolved transport");
        t.edge_kinds.assign(3, TransportKind::P2p);
        CHECK_THROWS_WITH(validate_topology(t), "expected 4 ring edges");
        t.edge_kinds.assign(4, TransportKind::P2p);
        t.local_rank_offset = 4;
        CHECK_THROWS_WITH(validate_topology(t), "local rank offset");
        t.local_rank_offset = 0;
        t.global_rank_count = 9;
        CHECK_THROWS_WITH(validate_topology(t), "within 1..8");
    }
    {   // edge resolution
        auto one_host = ranks(4, 4, true);
        for (auto k : resolve_edge_transports(TransportKind::Auto, one_host)) CHECK(k == TransportKind::P2p);
        for (auto k : resolve_edge_transports(TransportKind::Rdma, one_host)) CHECK(k == TransportKind::P2p);
        for (auto k : resolve_edge_transports(TransportKind::Socket, one_host)) CHECK(k == TransportKind::Socket);
        for (auto k : resolve_edge_transports(TransportKind::Shm, one_host)) CHECK(k == TransportKind::Shm);
        auto no_peer = ranks(4, 4, false);
        for (auto k : resolve_edge_transports(TransportKind::Auto, no_peer)) CHECK(k == TransportKind::Shm);
        CHECK_THROWS_WITH(resolve_edge_transports(TransportKind::P2p, no_peer), "available backend: shm");
        auto two_hosts = ranks(4, 2, true);  // edges 1->2 and 3->0 cross hosts
        auto mixed = resolve_edge_transports(TransportKind::Auto, two_hosts);
        CHECK(mixed[0] == TransportKind::P2p && mixed[1] == TransportKind::Socket && mixed[2] == TransportKind::P2p &&
              mixed[3] == TransportKind::Socket);
        auto rdma = resolve_edge_transports(TransportKind::Rdma, two_hosts);
        CHECK(rdma[1] == TransportKind::Rdma && rdma[0] == TransportKind::P2p);
        CHECK_THROWS_WITH(resolve_edge_transports(TransportKind::Shm, two_hosts), "edge 1 -> 2 crosses hosts");
        CHECK_THROWS_WITH(resolve_edge_transports(TransportKind::P2p, two_hosts), "available backend: socket");
        CHECK_THROWS_WITH(resolve_edge_transports(TransportKind::Mixed, one_host), "cannot be requested");
        RingTransportPlan plan{mixed};
        CHECK(plan.resolved_kind() == TransportKind::Mixed && plan.uses_p2p() && plan.uses(TransportKind::Socket) && !plan.all_p2p());
        RingTransportPlan uniform{resolve_edge_transports(TransportKind::Auto, one_host)};
        CHECK(uniform.resolved_kind() == TransportKind::P2p && uniform.all_p2p());
        CHECK(RingTransportPlan{}.resolved_kind() == TransportKind::Auto);
    }
    {   // two ranks of one host must not share a GPU
        auto v = ranks(2, 2, true);
        validate_unique_devices(v);
        v[1].uuid = v[0].uuid;
        CHECK_THROWS_WITH(validate_unique_devices(v), "same CUDA device");
        v[1].node_id = 999;  // same UUID bytes on another host: fine
        validate_unique_devices(v);
    }
    {   // names and parsers
        TransportKind t;
        CHECK(parse_transport("rdma", &t) && t == TransportKind::Rdma);
        CHECK(!parse_transport("mixed", &t) && !parse_transport("nvlink", &t));
        CHECK(std::string(transport_name(TransportKind::Mixed)) == "mixed");
        DType d;
        RedOp o;
        AlgoKind a;
        CHECK(parse_dtype("bf16", &d) && d == DType::BFloat16 && !parse_dtype("fp8", &d));
        CHECK(parse_redop("avg", &o) && o == RedOp::Avg && !parse_redop("prod", &o));
        CHECK(parse_algo("nvls", &a) && a == AlgoKind::Nvls && !parse_algo("tree", &a));
        auto s = make_sizes(262144, 67108864, 4);
        CHECK(s.size() == 5 && s.front() == 262144 && s.back() == 67108864);
        CHECK(make_sizes(1000, 5000, 4).back() == 5000);
        CHECK(all_reduce_busbw_gbs(100.0, 8) == 175.0 && gather_scatter_busbw_gbs(80.0, 8) == 70.0);
        CHECK(algbw_gbs(1000000, 1000.0) == 1.0);
    }
    {   // tuner
        unsetenv("NANO_NCCL_ALGO");
        unsetenv("NANO_NCCL_MAX_CTAS");
        unsetenv("NANO_NCCL_TUNER_FILE");
        Tuner t8(8, true);
        CHECK(t8.decide(CollectiveKind::AllReduce, 16 * 1024, RedOp::Sum).algo == AlgoKind::OneShot);
        CHECK(t8.decide(CollectiveKind::AllReduce, 4u << 20, RedOp::Sum).algo == AlgoKind::Nvls);
        CHECK(t8.decide(CollectiveKind::AllReduce, 64u << 20, RedOp::Sum).algo == AlgoKind::TwoShot);
        CHECK(t8.decide(CollectiveKind::AllReduce, 4u << 20, RedOp::Max).algo == AlgoKind::TwoShot);  // the switch only adds
        CHECK(Tuner(8, false).decide(CollectiveKind::AllReduce, 4u << 20, RedOp::Sum).algo == AlgoKind::TwoShot);
        CHECK(t8.decide(CollectiveKind::ReduceScatter, 1u << 20, RedOp::Min).algo == AlgoKind::OneShot);
        t8.set_forced_algo(AlgoKind::TwoShot);
        CHECK(t8.decide(CollectiveKind::AllReduce, 1024, RedOp::Sum).algo == AlgoKind::TwoShot);
        t8.set_forced_algo(AlgoKind::Ring);
        CHECK(t8.decide(CollectiveKind::AllGather, 1024, RedOp::Sum).algo == AlgoKind::Ring);
        t8.set_forced_algo(AlgoKind::Auto);
        // ReduceScatter / AllGather: the push kernels unless the zero-copy kernels are asked for and can apply
        CHECK(t8.decide(CollectiveKind::ReduceScatter, 1u << 20, RedOp::Sum).algo == AlgoKind::OneShot);
        CHECK(t8.decide(CollectiveKind::AllGather, 1u << 20, RedOp::Sum).algo == AlgoKind::OneShot);
        t8.set_forced_algo(AlgoKind::Nvls);
        CHECK(t8.decide(CollectiveKind::ReduceScatter, 1u << 20, RedOp::Avg).algo == AlgoKind::Nvls);
        CHECK(t8.decide(CollectiveKind::ReduceScatter, 1u << 20, RedOp::Max).algo == AlgoKind::OneShot);  // the switch only adds
        CHECK(t8.decide(CollectiveKind::AllGather, 1u << 20, RedOp::Sum).algo == AlgoKind::Nvls);
        t8.set_forced_algo(AlgoKind::Auto);
        {
            Tuner plain(8, false);   // no multicast: nothing to reduce in the switch, stores still work
            plain.set_forced_algo(AlgoKind::Nvls);
            CHECK(plain.decide(CollectiveKind::ReduceScatter, 1u << 20, RedOp::Sum).algo == AlgoKind::OneShot);
            CHECK(plain.decide(CollectiveKind::AllGather, 1u << 20, RedOp::Sum).algo == AlgoKind::Nvls);
        }
        t8.set_grid_override(7);
        CHECK(t8.decide(CollectiveKind::AllReduce, 1u << 20, RedOp::Sum).max_grid == 7);
        auto rules = Tuner::parse_rules("# comment\nall_reduce 8 1M twoshot 24\nall_gather 0 inf oneshot 48\n");
        CHECK(rules.size() == 2 && rules[0].max_bytes == (1u << 20) && rules[0].algo == AlgoKind::TwoShot && rules[1].grid == 48);
        CHECK_THROWS_WITH(Tuner::parse_rules("all_reduce 8 1M tree 24"), "unknown algorithm");
        CHECK_THROWS_WITH(Tuner::parse_rules("broadcast 8 1M ring 4"), "unknown collective");
        CHECK_THROWS_WITH(Tuner::parse_rules("all_reduce 8 1M ring 400"), "out of range");
        setenv("NANO_NCCL_ALGO", "bogus", 1);
        CHECK_THROWS_WITH(Tuner(2, true), "NANO_NCCL_ALGO");
        unsetenv("NANO_NCCL_ALGO");
    }
    {   // tile geometry: full coverage, limits respected, sub-slices even
        using dev::Family;
        for (Family fam : {Family::ArOneShot, Family::ArTwoShot, Family::ArNvls, Family::ReduceScatter, Family::AllGather}) {
            for (int n : {2, 3, 4, 8}) {
                for (std::size_t esz : {std::size_t{2}, std::size_t{4}}) {
                    for (std::size_t count : {std::size_t{1}, std::size_t{17}, std::size_t{16385}, std::size_t{5u << 20} + 3, std::size_t{1u << 28}}) {
                        for (int grid : {1, 16, 148}) {
                          for (std::size_t cap : {std::size_t{0}, std::size_t{65536}, std::size_t{200000}}) {
                            if (cap != 0 && count > (std::size_t{1} << 24)) continue;  // keeps the walk below short
                            const dev::Geometry g = dev::make_geometry(fam, count, esz, n, grid, cap == 65536, cap);
                            if (cap != 0) CHECK(g.tile_elems * esz <= std::max<std::size_t>(cap, 2 * n * 16));
                            CHECK(g.grid >= 1 && g.grid <= grid);
                            CHECK(g.tile_elems % (2 * static_cast<std::size_t>(n) * (16 / esz)) == 0);
                            CHECK(g.tile_elems * esz <= dev::max_tile_bytes(fam, n));
                            CHECK(static_cast<std::size_t>(g.grid) * g.region_elems >= count);
                            if (fam == Family::ArTwoShot) CHECK(g.slot_bytes * n <= dev::kHalfBytes / 2);
                            else if (fam != Family::ArNvls) CHECK(g.slot_bytes * n <= dev::kHalfBytes);
                            // the tiles of every CTA cover its region exactly once, in order
                            std::size_t cursor = 0;
                            for (int b = 0; b < g.grid; ++b) {
                                CHECK(cursor == std::min(count, static_cast<std::size_t>(b) * g.region_elems));
                                for (int it = 0; it < g.iters; ++it) {
                                    std::size_t t0, len;
                                    dev::tile_range_of(g, count, static_cast<unsigned>(b), it, &t0, &len);
                                    if (len == 0) continue;
                                    CHECK(t0 == cursor && len <= g.tile_elems);
                                    cursor += len;
                                }
                            }
                            CHECK(cursor == count);
                          }
                        }
                    }
                }
            }
        }
    }
    {   // GEMM tile width: whole waves of CTAs times the width decide
        unsetenv("NANO_NCCL_GEMM_BN");
        CHECK(gemm_pick_tile_width(64, 1792, 148) == 256);           // the default is the full tile
        setenv("NANO_NCCL_GEMM_BN", "auto", 1);
        CHECK(gemm_pick_tile_width(64, 1792, 148) == 224);           // 512 tiles: 4 waves x 224 beats 4 x 256
        CHECK(gemm_pick_tile_width(64, 4096, 148) == 256);           // 1024 tiles: 7 waves x 256 is the least
        CHECK(gemm_pick_tile_width(64, 1792, 148, 64) == 192);       // boxes of 64 columns: 5 waves x 192 beats 4 x 256
        setenv("NANO_NCCL_GEMM_BN", "192", 1);
        CHECK(gemm_pick_tile_width(64, 1792, 148) == 192);
        setenv("NANO_NCCL_GEMM_BN", "200", 1);
        CHECK_THROWS_WITH(gemm_pick_tile_width(64, 1792, 148), "NANO_NCCL_GEMM_BN");
        setenv("NANO_NCCL_GEMM_BN", "224", 1);
        CHECK_THROWS_WITH(gemm_pick_tile_width(64, 1792, 148, 64), "multiple of 64");
        unsetenv("NANO_NCCL_GEMM_BN");
    }
    {   // split of the last, partly filled round of a persistent GEMM into narrow column pieces
        unsetenv("NANO_NCCL_GEMM_TAIL");
        GemmTailSplit t = gemm_pick_tail_split(448, 148, 256);      // 8192 x 1792: 4 tiles left -> 32 pieces of 32 columns
        CHECK(t.first_tile == 444 && t.piece_bn == 32);
        t = gemm_pick_tail_split(512, 148, 256);                    // 4096^2: 68 left -> 136 pieces of 128 columns
        CHECK(t.first_tile == 444 && t.piece_bn == 128);
        t = gemm_pick_tail_split(462, 148, 256);                    // 18 left: 8 pieces each fit (144), so 32 columns
        CHECK(t.first_tile == 444 && t.piece_bn == 32);
        t = gemm_pick_tail_split(474, 148, 256);                    // 30 left: 4 pieces each (120) -> 64 columns
        CHECK(t.first_tile == 444 && t.piece_bn == 64);
        t = gemm_pick_tail_split(2048, 148, 256);                   // 124 left: more than half the CTAs, no split
        CHECK(t.first_tile == 2048 && t.piece_bn == 0);
        t = gemm_pick_tail_split(1024, 128, 256);                   // whole rounds
        CHECK(t.piece_bn == 0);
        t = gemm_pick_tail_split(100, 148, 256);                    // a single round
        CHECK(t.piece_bn == 0);
        t = gemm_pick_tail_split(452, 148, 224);                    // 224 columns: only 32 divides it
        CHECK(t.first_tile == 444 && t.piece_bn == 32);
        setenv("NANO_NCCL_GEMM_TAIL", "0", 1);
        CHECK(gemm_pick_tail_split(448, 148, 256).piece_bn == 0);
        unsetenv("NANO_NCCL_GEMM_TAIL");
    }
    std::printf("topology_tuner_test ok\n");
    return 0;
}
