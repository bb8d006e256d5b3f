// Host-side checks of the two visiting orders the kernels share (no GPU): which output tile a CTA takes at
// step i (tile_coord, pair_tile_coord) and which (16-row chunk, K segment) a quantise or pusher worker takes
// at step i (item_coord).  They stand in for the reference's scheduling helpers
// (include/catccos/catccos.hpp:148-176, include/catccos/dgemm/block/block_swizzle_allgather.hpp:59-90): the
// contract is "every unit exactly once; this rank's own rows first, then the peers in ring order, slice by
// slice (or, for a quantiser that sends every item to all ranks at once, slice by slice over all ranks with
// the own slice leading); inside a send group the K segments in order".  Exit code 0 = pass.
#include <cstdio>
#include <set>
#include <vector>

#include "../../catccos_b200/csrc/mx_gemm_pair.cuh"

using namespace catccos;

#define EXPECT(cond)                                                   \
    do {                                                               \
        if (!(cond)) {                                                 \
            std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); \
            return 1;                                                  \
        }                                                              \
    } while (0)

static int check_tiles(uint32_t world, uint32_t rank, uint32_t m_local, uint32_t n, bool pair, bool own_first)
{
    GemmParams p = {};
    p.own_first = own_first ? 1u : 0u;
    uint32_t flag_word = 0;
    p.flags = &flag_word;  // gated launch: arrival order
    p.world = world;
    p.rank = rank;
    p.m_local = m_local;
    p.Mg = world * m_local;
    p.N = n;
    const uint32_t bm = pair ? kPairBlockM : kGemmBlockM;
    const uint32_t m_tiles = (p.Mg + bm - 1) / bm, n_tiles = (n + 255) / 256;
    std::set<std::pair<uint32_t, uint32_t>> seen;
    uint32_t prev_src_pos = 0, prev_slice = 0;
    for (uint32_t i = 0; i < m_tiles * n_tiles; ++i) {
        const TileCoord t = pair ? pair_tile_coord(i, n_tiles, m_tiles, p) : tile_coord(i, n_tiles, m_tiles, p);
        EXPECT(t.m_tile < m_tiles && t.n_tile < n_tiles);
        EXPECT(seen.insert({t.m_tile, t.n_tile}).second);  // every tile exactly once
        EXPECT(t.n_tile == i % n_tiles);                    // n runs fastest: neighbours share an A panel
        if (m_local % bm == 0 && world > 1) {
            const uint32_t tps = m_local / bm;
            const uint32_t src = t.m_tile / tps, slice = t.m_tile % tps;
            const uint32_t src_pos = (src + world - rank) % world;  // 0 = own shard, 1 = next rank in the ring, ...
            if (!own_first) {
                // slice by slice over all ranks; inside a slice this rank first, then the ring behind it
                const uint32_t mo = i / n_tiles;
                EXPECT(slice == mo / world && src_pos == mo % world);
            } else if (i < tps * n_tiles) {
                EXPECT(src == rank);  // this rank's own rows first: they need no transfer
            } else {
                EXPECT(src != rank);
                // then slice by slice, and inside a slice the peers in ring order behind this rank
                if (i > tps * n_tiles && t.n_tile == 0) {
                    EXPECT(slice > prev_slice || (slice == prev_slice && src_pos > prev_src_pos));
                }
                prev_slice = slice;
                prev_src_pos = src_pos;
            }
        }
    }
    EXPECT(seen.size() == (size_t)m_tiles * n_tiles);
    return 0;
}

static int check_items(uint32_t chunks, uint32_t segs, uint32_t group_chunks, const std::vector<uint8_t>& order)
{
    std::set<std::pair<uint32_t, uint32_t>> seen;
    uint32_t prev_group = 0, prev_pos = 0;
    for (uint32_t item = 0; item < chunks * segs; ++item) {
        uint32_t chunk = 0, seg = 0;
        item_coord(item, chunks, segs, group_chunks, order.data(), (uint32_t)order.size(), chunk, seg);
        EXPECT(chunk < chunks && seg < segs);
        EXPECT(seen.insert({chunk, seg}).second);  // every (chunk, segment) exactly once
        const uint32_t gc = (group_chunks == 0 || group_chunks > chunks) ? chunks : group_chunks;
        const uint32_t group = chunk / gc;
        uint32_t pos = seg;
        if (order.size() == segs) {
            for (uint32_t i = 0; i < segs; ++i) {
                if (order[i] == seg) pos = i;
            }
        }
        if (item > 0) {
            // groups follow one another; inside a group the segments follow the visiting order
            EXPECT(group > prev_group || (group == prev_group && pos >= prev_pos));
        }
        prev_group = group;
        prev_pos = pos;
    }
    EXPECT(seen.size() == (size_t)chunks * segs);
    return 0;
}

int main()
{
    for (bool pair : {false, true}) {
        for (uint32_t world : {1u, 2u, 4u, 8u}) {
            for (uint32_t rank = 0; rank < world; ++rank) {
                for (bool own_first : {true, false}) {
                    if (check_tiles(world, rank, 1024, 2304, pair, own_first) != 0) return 1;  // the prefill shape
                    if (check_tiles(world, rank, 4096, 3456, pair, own_first) != 0) return 1;  // the outlier shape
                    if (check_tiles(world, rank, 16, 4096, pair, own_first) != 0) return 1;    // decode: shards smaller than a tile
                    if (check_tiles(world, rank, 190, 272, pair, own_first) != 0) return 1;    // ragged
                }
            }
        }
    }
    if (check_items(64, 7, 0, {}) != 0) return 1;
    if (check_items(64, 7, 16, {}) != 0) return 1;
    if (check_items(63, 5, 16, {}) != 0) return 1;  // last group short
    if (check_items(1, 14, 0, {0, 2, 4, 6, 8, 10, 12, 1, 3, 5, 7, 9, 11, 13}) != 0) return 1;  // split-K round-robin
    if (check_items(256, 3, 16, {}) != 0) return 1;
    std::printf("PASS\n");
    return 0;
}
