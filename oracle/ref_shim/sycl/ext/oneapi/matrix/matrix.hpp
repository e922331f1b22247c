// joint_matrix on the host, for the reference's matrix-unit kernels run as a check on the oracle. Test infrastructure only.
//
// The shapes those kernels use and nothing else: A [M][16] half row-major, B [16][16] half in the packed ("VNNI") layout
// - memory word (k / 2, n) holds elements (k, n) and (k + 1, n), low half first -, the accumulator [M][16] float, a
// sub-group of 16. Every work-item holds a whole copy of A and B (they are only ever loaded), and of the accumulator the
// column of its own lane: element (row e, column lane) is the lane's e-th element, the ownership the kernels' row
// rescales through joint_matrix_apply rely on. joint_matrix_mad is D[r][lane] = C[r][lane] + sum over k = 0 .. 15, in
// that order, of A[r][k] B[k][lane], the products and sums in fp32 (a half times a half is exact in fp32). The order
// in which the matrix unit itself adds the 16 products is not published; this is the plain one.
#pragma once
#include <sycl/sycl.hpp>

namespace sycl {
namespace ext {
namespace oneapi {
namespace experimental {
namespace matrix {

enum class use { a, b, accumulator };
enum class layout { row_major, col_major, ext_intel_packed, dynamic };

template <class Group, class T, use U, size_t R, size_t C, layout L = layout::dynamic>
struct joint_matrix {
    T v[R][C];
};

namespace detail {
inline int lane_of(const sycl::sub_group& sg) { return (int) sg.get_local_linear_id(); }
}  // namespace detail

template <class T, size_t R, size_t C, layout L>
void joint_matrix_load(const sycl::sub_group&, joint_matrix<sycl::sub_group, T, use::a, R, C, L>& m, const T* p, size_t stride) {
    static_assert(L == layout::row_major, "A: row-major");
    for (size_t r = 0; r < R; ++r)
        for (size_t c = 0; c < C; ++c) m.v[r][c] = p[r * stride + c];
}
template <class T, size_t R, size_t C, layout L>
void joint_matrix_load(const sycl::sub_group&, joint_matrix<sycl::sub_group, T, use::b, R, C, L>& m, const T* p, size_t stride) {
    static_assert(L == layout::ext_intel_packed && sizeof(T) == 2, "B: 16-bit elements, packed in pairs of rows");
    for (size_t k = 0; k < R; ++k)
        for (size_t n = 0; n < C; ++n) m.v[k][n] = p[(k / 2) * stride + n * 2 + (k & 1)];
}
template <class T, use U, size_t R, size_t C, layout L, class V>
void joint_matrix_fill(const sycl::sub_group&, joint_matrix<sycl::sub_group, T, U, R, C, L>& m, V x) {
    for (size_t r = 0; r < R; ++r)
        for (size_t c = 0; c < C; ++c) m.v[r][c] = (T) x;
}
template <class TA, class TB, size_t M, size_t K, size_t N, layout LA, layout LB>
void joint_matrix_mad(const sycl::sub_group& sg, joint_matrix<sycl::sub_group, float, use::accumulator, M, N>& d,
                      const joint_matrix<sycl::sub_group, TA, use::a, M, K, LA>& a, const joint_matrix<sycl::sub_group, TB, use::b, K, N, LB>& b,
                      const joint_matrix<sycl::sub_group, float, use::accumulator, M, N>& c) {
    static_assert(N == 16, "a column a lane");
    const int n = detail::lane_of(sg);
    for (size_t r = 0; r < M; ++r) {
        float acc = c.v[r][n];
        for (size_t k = 0; k < K; ++k) acc += (float) a.v[r][k] * (float) b.v[k][n];
        d.v[r][n] = acc;
    }
}
template <size_t R, size_t C>
void joint_matrix_store(const sycl::sub_group& sg, const joint_matrix<sycl::sub_group, float, use::accumulator, R, C>& m, float* p, size_t stride, layout l) {
    static_assert(C == 16, "a column a lane");
    const int n = detail::lane_of(sg);
    for (size_t r = 0; r < R; ++r) {
        if (l == layout::row_major) p[r * stride + n] = m.v[r][n];
        else p[n * stride + r] = m.v[r][n];
    }
}
// the lane's own elements, in the order of their rows
template <size_t R, size_t C, class F>
void joint_matrix_apply(const sycl::sub_group& sg, joint_matrix<sycl::sub_group, float, use::accumulator, R, C>& m, F&& f) {
    static_assert(C == 16, "a column a lane");
    const int n = detail::lane_of(sg);
    for (size_t r = 0; r < R; ++r) f(m.v[r][n]);
}

}  // namespace matrix
}  // namespace experimental
}  // namespace oneapi
}  // namespace ext
}  // namespace sycl
