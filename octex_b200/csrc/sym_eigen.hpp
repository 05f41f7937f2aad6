// Eigen-decomposition of a real symmetric matrix on the host (fp64), for the sample PCA of the index
// builder: the reference hands its scatter matrix to cuSOLVER (hpdic/octex,
// cpp/src/neighbors/octex/detail/build_setup.cuh:82-86); the matrix is dim x dim, so a plain
// Householder + QL solver on the host takes a second or two at most.
#pragma once

#include "common.hpp"

#include <algorithm>
#include <cmath>
#include <vector>

namespace octex_b200 {

/// Eigenvalues (ascending) and eigenvectors (columns of v, stored row major [n, n]) of the
/// symmetric matrix a [n, n] (destroyed): Householder reduction to tridiagonal form, then the QL
/// algorithm with implicit shifts. Host code, fp64; n is a dimension (at most a few thousand).
inline void symmetric_eigen(std::vector<double>& a, int n, std::vector<double>& d, std::vector<double>& v)
{
  std::vector<double> e(n, 0.0);
  d.assign(n, 0.0);
  auto A = [&](int i, int j) -> double& { return a[static_cast<size_t>(i) * n + j]; };
  // reduction to tridiagonal form; a is overwritten with the orthogonal transformation
  for (int i = n - 1; i > 0; i--) {
    const int l = i - 1;
    double h = 0.0, scale = 0.0;
    if (l > 0) {
      for (int k = 0; k <= l; k++)
        scale += std::fabs(A(i, k));
      if (scale == 0.0) {
        e[i] = A(i, l);
      } else {
        for (int k = 0; k <= l; k++) {
          A(i, k) /= scale;
          h += A(i, k) * A(i, k);
        }
        double f = A(i, l);
        double g = f >= 0.0 ? -std::sqrt(h) : std::sqrt(h);
        e[i]     = scale * g;
        h -= f * g;
        A(i, l) = f - g;
        f       = 0.0;
        for (int j = 0; j <= l; j++) {
          A(j, i) = A(i, j) / h;
          g       = 0.0;
          for (int k = 0; k <= j; k++)
            g += A(j, k) * A(i, k);
          for (int k = j + 1; k <= l; k++)
            g += A(k, j) * A(i, k);
          e[j] = g / h;
          f += e[j] * A(i, j);
        }
        const double hh = f / (h + h);
        for (int j = 0; j <= l; j++) {
          f    = A(i, j);
          e[j] = g = e[j] - hh * f;
          for (int k = 0; k <= j; k++)
            A(j, k) -= f * e[k] + g * A(i, k);
        }
      }
    } else {
      e[i] = A(i, l);
    }
    d[i] = h;
  }
  d[0] = 0.0;
  e[0] = 0.0;
  for (int i = 0; i < n; i++) {
    const int l = i - 1;
    if (d[i] != 0.0) {
      for (int j = 0; j <= l; j++) {
        double g = 0.0;
        for (int k = 0; k <= l; k++)
          g += A(i, k) * A(k, j);
        for (int k = 0; k <= l; k++)
          A(k, j) -= g * A(k, i);
      }
    }
    d[i]    = A(i, i);
    A(i, i) = 1.0;
    for (int j = 0; j <= l; j++)
      A(j, i) = A(i, j) = 0.0;
  }
  // QL with implicit shifts on (d, e); the transformation accumulates in a
  for (int i = 1; i < n; i++)
    e[i - 1] = e[i];
  e[n - 1] = 0.0;
  for (int l = 0; l < n; l++) {
    int iter = 0, m;
    do {
      for (m = l; m < n - 1; m++) {
        const double dd = std::fabs(d[m]) + std::fabs(d[m + 1]);
        if (std::fabs(e[m]) <= 2.3e-16 * dd) break;
      }
      if (m != l) {
        OCTEX_EXPECTS(iter++ < 200, "octex: the eigenvalue iteration of the sample PCA did not converge");
        double g = (d[l + 1] - d[l]) / (2.0 * e[l]);
        double r = std::hypot(g, 1.0);
        g        = d[m] - d[l] + e[l] / (g + (g >= 0.0 ? std::fabs(r) : -std::fabs(r)));
        double s = 1.0, c = 1.0, p = 0.0;
        int i;
        for (i = m - 1; i >= l; i--) {
          double f = s * e[i], b = c * e[i];
          e[i + 1] = r = std::hypot(f, g);
          if (r == 0.0) {
            d[i + 1] -= p;
            e[m] = 0.0;
            break;
          }
          s        = f / r;
          c        = g / r;
          g        = d[i + 1] - p;
          r        = (d[i] - g) * s + 2.0 * c * b;
          d[i + 1] = g + (p = s * r);
          g        = c * r - b;
          for (int k = 0; k < n; k++) {
            f           = A(k, i + 1);
            A(k, i + 1) = s * A(k, i) + c * f;
            A(k, i)     = c * A(k, i) - s * f;
          }
        }
        if (r == 0.0 && i >= l) continue;
        d[l] -= p;
        e[l] = g;
        e[m] = 0.0;
      }
    } while (m != l);
  }
  // ascending order
  std::vector<int> order(n);
  for (int i = 0; i < n; i++)
    order[i] = i;
  std::sort(order.begin(), order.end(), [&](int x, int y) { return d[x] < d[y]; });
  std::vector<double> ds(n);
  v.assign(static_cast<size_t>(n) * n, 0.0);
  for (int j = 0; j < n; j++) {
    ds[j] = d[order[j]];
    for (int k = 0; k < n; k++)
      v[static_cast<size_t>(k) * n + j] = A(k, order[j]);
  }
  d.swap(ds);
}

}  // namespace octex_b200
