// Triangle mesh simplification by quadric-error edge collapses (host side of the image-to-3D pipeline).
//
// The reference decimates extracted meshes on the host with inherited plane quadrics and manifold link checks
// (src/sparse.rs: Quadric :274-382, EdgeQueue :411-530, MeshDecimator :534-1000). This is an independent
// implementation of the same scheme:
//   * every vertex carries the sum of the plane quadrics of its faces (unit normals, FP64);
//   * an edge (a, b) costs the smallest error of Q_a + Q_b over a few candidate points (the quadric's stationary point
//     when the system is well conditioned, the minimum on the segment, the end points, the mid point);
//   * a binary heap with per-vertex stamps orders the edges, stale entries are skipped when popped;
//   * a collapse is refused when the link condition fails (the common neighbours of a and b must be exactly the
//     vertices opposite the edge) or when a surviving face would flip or degenerate.
// Outputs the compacted mesh and, per output face / vertex, the index of the input face / vertex it descends from.
#include <algorithm>
#include <array>
#include <cmath>
#include <cstdint>
#include <iterator>
#include <queue>
#include <vector>

namespace {

using Vec3 = std::array<double, 3>;

inline Vec3 sub(const Vec3& a, const Vec3& b) { return {a[0] - b[0], a[1] - b[1], a[2] - b[2]}; }
inline double dot(const Vec3& a, const Vec3& b) { return a[0] * b[0] + a[1] * b[1] + a[2] * b[2]; }
inline Vec3 cross(const Vec3& a, const Vec3& b) {
  return {a[1] * b[2] - a[2] * b[1], a[2] * b[0] - a[0] * b[2], a[0] * b[1] - a[1] * b[0]};
}

// symmetric 4x4 form: xx xy xz xw yy yz yw zz zw ww
struct Quadric {
  double q[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
  void add_plane(double a, double b, double c, double d) {
    const double p[4] = {a, b, c, d};
    int k = 0;
    for (int i = 0; i < 4; ++i)
      for (int j = i; j < 4; ++j) q[k++] += p[i] * p[j];
  }
  Quadric operator+(const Quadric& o) const {
    Quadric r;
    for (int i = 0; i < 10; ++i) r.q[i] = q[i] + o.q[i];
    return r;
  }
  double energy(const Vec3& v) const {
    const double x = v[0], y = v[1], z = v[2];
    return q[0] * x * x + 2 * q[1] * x * y + 2 * q[2] * x * z + 2 * q[3] * x + q[4] * y * y + 2 * q[5] * y * z + 2 * q[6] * y +
           q[7] * z * z + 2 * q[8] * z + q[9];
  }
  Vec3 apply(const Vec3& v) const {
    return {q[0] * v[0] + q[1] * v[1] + q[2] * v[2], q[1] * v[0] + q[4] * v[1] + q[5] * v[2], q[2] * v[0] + q[5] * v[1] + q[7] * v[2]};
  }
  // solves A x = -b by Gauss-Jordan with partial pivoting; refuses nearly singular systems
  bool stationary(Vec3* out) const {
    double a[3][4] = {{q[0], q[1], q[2], -q[3]}, {q[1], q[4], q[5], -q[6]}, {q[2], q[5], q[7], -q[8]}};
    const double scale = std::max({std::fabs(q[0]), std::fabs(q[4]), std::fabs(q[7])});
    for (int c = 0; c < 3; ++c) {
      int piv = c;
      for (int r = c + 1; r < 3; ++r)
        if (std::fabs(a[r][c]) > std::fabs(a[piv][c])) piv = r;
      if (std::fabs(a[piv][c]) <= 1e-12 * scale) return false;
      if (piv != c) std::swap(a[piv], a[c]);
      const double d = a[c][c];
      for (int k = c; k < 4; ++k) a[c][k] /= d;
      for (int r = 0; r < 3; ++r) {
        if (r == c) continue;
        const double f = a[r][c];
        for (int k = c; k < 4; ++k) a[r][k] -= f * a[c][k];
      }
    }
    *out = {a[0][3], a[1][3], a[2][3]};
    return std::isfinite((*out)[0]) && std::isfinite((*out)[1]) && std::isfinite((*out)[2]);
  }
  Vec3 on_segment(const Vec3& a, const Vec3& b) const {
    const Vec3 d = sub(b, a);
    const Vec3 qa = apply(a);
    const double num = dot(d, {qa[0] + q[3], qa[1] + q[6], qa[2] + q[8]});
    const double den = dot(d, apply(d));
    const double t = den > 0.0 ? std::min(1.0, std::max(0.0, -num / den)) : 0.0;
    return {a[0] + t * d[0], a[1] + t * d[1], a[2] + t * d[2]};
  }
};

struct Entry {
  double cost;
  int a, b;
  uint32_t stamp_a, stamp_b;
  bool operator<(const Entry& o) const {          // min-heap on (cost, a, b)
    if (cost != o.cost) return cost > o.cost;
    if (a != o.a) return a > o.a;
    return b > o.b;
  }
};

struct Decimator {
  std::vector<Vec3> pos;
  std::vector<std::array<int, 3>> tri;
  std::vector<char> live_face, live_vertex;
  std::vector<std::vector<int>> faces_of;         // incident live faces (may hold dead ones; filtered on use)
  std::vector<Quadric> quad;
  std::vector<uint32_t> stamp;
  std::priority_queue<Entry> heap;
  int live_faces = 0;

  bool face_normal(const std::array<int, 3>& t, Vec3* n) const {
    const Vec3 c = cross(sub(pos[t[1]], pos[t[0]]), sub(pos[t[2]], pos[t[0]]));
    const double len = std::sqrt(dot(c, c));
    if (!(len > 0.0) || !std::isfinite(len)) return false;
    *n = {c[0] / len, c[1] / len, c[2] / len};
    return true;
  }

  void best_point(int a, int b, Vec3* point, double* cost) const {
    const Quadric q = quad[a] + quad[b];
    Vec3 cand[5];
    int n = 0;
    Vec3 s;
    if (q.stationary(&s)) cand[n++] = s;
    cand[n++] = q.on_segment(pos[a], pos[b]);
    cand[n++] = pos[a];
    cand[n++] = pos[b];
    cand[n++] = {(pos[a][0] + pos[b][0]) * 0.5, (pos[a][1] + pos[b][1]) * 0.5, (pos[a][2] + pos[b][2]) * 0.5};
    *cost = INFINITY;
    for (int i = 0; i < n; ++i) {
      const double e = std::max(0.0, q.energy(cand[i]));
      if (e < *cost) { *cost = e; *point = cand[i]; }
    }
  }

  void push_edge(int a, int b) {
    if (a > b) std::swap(a, b);
    Vec3 p;
    double c;
    best_point(a, b, &p, &c);
    heap.push({c, a, b, stamp[a], stamp[b]});
  }

  void neighbours(int v, std::vector<int>* out) const {
    out->clear();
    for (int f : faces_of[v]) {
      if (!live_face[f]) continue;
      for (int k = 0; k < 3; ++k)
        if (tri[f][k] != v) out->push_back(tri[f][k]);
    }
    std::sort(out->begin(), out->end());
    out->erase(std::unique(out->begin(), out->end()), out->end());
  }

  bool link_ok(int a, int b) const {
    std::vector<int> na, nb, common, opposite;
    neighbours(a, &na);
    neighbours(b, &nb);
    std::set_intersection(na.begin(), na.end(), nb.begin(), nb.end(), std::back_inserter(common));
    for (int f : faces_of[a]) {
      if (!live_face[f]) continue;
      const auto& t = tri[f];
      if (t[0] != b && t[1] != b && t[2] != b) continue;
      for (int k = 0; k < 3; ++k)
        if (t[k] != a && t[k] != b) opposite.push_back(t[k]);
    }
    std::sort(opposite.begin(), opposite.end());
    // an edge with more than two faces, or a face listed twice, is not collapsed
    if (opposite.empty() || opposite.size() > 2 || std::adjacent_find(opposite.begin(), opposite.end()) != opposite.end()) return false;
    return common == opposite;
  }

  bool geometry_ok(int a, int b, const Vec3& p) const {
    for (int v : {a, b}) {
      for (int f : faces_of[v]) {
        if (!live_face[f]) continue;
        std::array<int, 3> t = tri[f];
        const bool has_a = t[0] == a || t[1] == a || t[2] == a, has_b = t[0] == b || t[1] == b || t[2] == b;
        if (has_a && has_b) continue;                          // disappears with the edge
        Vec3 before;
        if (!face_normal(t, &before)) continue;
        Vec3 q[3];
        for (int k = 0; k < 3; ++k) q[k] = (t[k] == a || t[k] == b) ? p : pos[t[k]];
        const Vec3 c = cross(sub(q[1], q[0]), sub(q[2], q[0]));
        const double len = std::sqrt(dot(c, c));
        if (!(len > 1e-300) || dot(c, before) <= 0.2 * len) return false;   // flipped, or turned by more than ~78 degrees
      }
    }
    return true;
  }

  void collapse(int a, int b, const Vec3& p) {
    pos[a] = p;
    quad[a] = quad[a] + quad[b];
    for (int f : faces_of[b]) {
      if (!live_face[f]) continue;
      auto& t = tri[f];
      const bool has_a = t[0] == a || t[1] == a || t[2] == a;
      if (has_a) {
        live_face[f] = 0;
        --live_faces;
        continue;
      }
      for (int k = 0; k < 3; ++k)
        if (t[k] == b) t[k] = a;
      faces_of[a].push_back(f);
    }
    faces_of[b].clear();
    live_vertex[b] = 0;
    auto& fa = faces_of[a];
    fa.erase(std::remove_if(fa.begin(), fa.end(), [&](int f) { return !live_face[f]; }), fa.end());
    ++stamp[a];
    ++stamp[b];
    std::vector<int> nb;
    neighbours(a, &nb);
    for (int v : nb) push_edge(a, v);
  }
};

}  // namespace

extern "C" {

// vertices [n, 3] f32, faces [m, 3] i32 -> at most `target` faces. out_vertices [n, 3], out_faces [m, 3], face_map [m],
// vertex_map [n] are caller buffers of the input sizes; counts = {vertices out, faces out, collapses done}.
// Returns 0, or -1 for invalid input.
__attribute__((visibility("default"))) int ff_mesh_simplify(const float* vertices, int n, const int* faces, int m, int target, float* out_vertices, int* out_faces,
                     int* face_map, int* vertex_map, int* counts) {
  if (!vertices || !faces || n <= 0 || m <= 0 || target <= 0 || !out_vertices || !out_faces || !face_map || !vertex_map || !counts) return -1;
  Decimator d;
  d.pos.resize(n);
  for (int i = 0; i < n; ++i) {
    d.pos[i] = {vertices[3 * i], vertices[3 * i + 1], vertices[3 * i + 2]};
    if (!std::isfinite(d.pos[i][0]) || !std::isfinite(d.pos[i][1]) || !std::isfinite(d.pos[i][2])) return -1;
  }
  d.tri.resize(m);
  d.live_face.assign(m, 1);
  d.live_vertex.assign(n, 0);
  d.faces_of.assign(n, {});
  d.quad.assign(n, Quadric());
  d.stamp.assign(n, 0);
  d.live_faces = m;
  for (int f = 0; f < m; ++f) {
    for (int k = 0; k < 3; ++k) {
      const int v = faces[3 * f + k];
      if (v < 0 || v >= n) return -1;
      d.tri[f][k] = v;
    }
    const auto& t = d.tri[f];
    if (t[0] == t[1] || t[1] == t[2] || t[0] == t[2]) {        // degenerate input faces are dropped
      d.live_face[f] = 0;
      --d.live_faces;
      continue;
    }
    for (int k = 0; k < 3; ++k) {
      d.faces_of[t[k]].push_back(f);
      d.live_vertex[t[k]] = 1;
    }
    Vec3 nrm;
    if (d.face_normal(t, &nrm)) {
      const double w = -dot(nrm, d.pos[t[0]]);
      for (int k = 0; k < 3; ++k) d.quad[t[k]].add_plane(nrm[0], nrm[1], nrm[2], w);
    }
  }
  std::vector<int> nb;
  for (int v = 0; v < n; ++v) {
    if (!d.live_vertex[v]) continue;
    d.neighbours(v, &nb);
    for (int u : nb)
      if (u > v) d.push_edge(v, u);
  }
  int collapses = 0;
  while (d.live_faces > target && !d.heap.empty()) {
    const Entry e = d.heap.top();
    d.heap.pop();
    if (!d.live_vertex[e.a] || !d.live_vertex[e.b] || d.stamp[e.a] != e.stamp_a || d.stamp[e.b] != e.stamp_b) continue;
    Vec3 p;
    double cost;
    d.best_point(e.a, e.b, &p, &cost);
    if (!d.link_ok(e.a, e.b) || !d.geometry_ok(e.a, e.b, p)) continue;    // comes back when a neighbour changes
    d.collapse(e.a, e.b, p);
    ++collapses;
  }
  std::vector<int> remap(n, -1);
  int nv = 0, nf = 0;
  for (int f = 0; f < m; ++f) {
    if (!d.live_face[f]) continue;
    for (int k = 0; k < 3; ++k) {
      const int v = d.tri[f][k];
      if (remap[v] < 0) {
        remap[v] = nv;
        vertex_map[nv] = v;
        for (int j = 0; j < 3; ++j) out_vertices[3 * nv + j] = static_cast<float>(d.pos[v][j]);
        ++nv;
      }
      out_faces[3 * nf + k] = remap[v];
    }
    face_map[nf++] = f;
  }
  counts[0] = nv;
  counts[1] = nf;
  counts[2] = collapses;
  return 0;
}

}  // extern "C"
