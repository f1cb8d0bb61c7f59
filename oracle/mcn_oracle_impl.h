/* Body of the plain-C restatement, included once per element type.
 *
 * TEST INFRASTRUCTURE ONLY (see mcn_oracle.c).  Before inclusion define
 *   T       element type (float or double)
 *   FN(x)   name mangler, e.g. x##_f32
 * All tensors are MATLAB-order H x W x C x N: element (h,w,c,n) lives at
 * h + H*(w + W*(c + C*n)) (reference matlab/src/bits/data.cu:498-505).
 * Paths cited below are relative to the reference's matlab/src/bits/.
 */

#define IDX4(h, w, c, n, H, W, C) ((size_t)(h) + (size_t)(H) * ((size_t)(w) + (size_t)(W) * ((size_t)(c) + (size_t)(C) * (size_t)(n))))

/* ------------------------------------------------------------------ */
/* Convolution (nnconv.cu:71-157 forward, :163-317 backward)           */
/* ------------------------------------------------------------------ */

/* Patch matrix of one image (impl/im2row_cpu.cpp:52-163): column-major
 * (Ho*Wo) x (FH*FW*C); row = ho + Ho*wo, column = fh + FH*(fw + FW*c);
 * taps outside the image are zero. */
static void FN(im2row)(T* patches, T const* x, int H, int W, int C, int FH, int FW, int Ho, int Wo,
                       int sy, int sx, int pt, int pl, int dy, int dx)
{
  size_t P = (size_t)Ho * Wo;
  for (int c = 0; c < C; ++c)
    for (int fw = 0; fw < FW; ++fw)
      for (int fh = 0; fh < FH; ++fh) {
        T* col = patches + P * ((size_t)fh + FH * ((size_t)fw + (size_t)FW * c));
        for (int wo = 0; wo < Wo; ++wo) {
          int w = wo * sx + fw * dx - pl;
          for (int ho = 0; ho < Ho; ++ho) {
            int h = ho * sy + fh * dy - pt;
            col[ho + (size_t)Ho * wo] =
                (h >= 0 && h < H && w >= 0 && w < W) ? x[h + (size_t)H * (w + (size_t)W * c)] : (T)0;
          }
        }
      }
}

/* Transpose of the above (impl/im2row_cpu.cpp:169-230): zero the image, then
 * add every patch-matrix entry back to the pixel it was taken from, columns
 * in ascending order, rows in ascending order within a column. */
static void FN(row2im)(T* x, T const* patches, int H, int W, int C, int FH, int FW, int Ho, int Wo,
                       int sy, int sx, int pt, int pl, int dy, int dx)
{
  size_t P = (size_t)Ho * Wo;
  memset(x, 0, sizeof(T) * (size_t)H * W * C);
  for (int c = 0; c < C; ++c)
    for (int fw = 0; fw < FW; ++fw)
      for (int fh = 0; fh < FH; ++fh) {
        T const* col = patches + P * ((size_t)fh + FH * ((size_t)fw + (size_t)FW * c));
        for (int wo = 0; wo < Wo; ++wo) {
          int w = wo * sx + fw * dx - pl;
          if (w < 0 || w >= W) continue;
          for (int ho = 0; ho < Ho; ++ho) {
            int h = ho * sy + fh * dy - pt;
            if (h < 0 || h >= H) continue;
            x[h + (size_t)H * (w + (size_t)W * c)] += col[ho + (size_t)Ho * wo];
          }
        }
      }
}

/* shape = {H,W,C,N,FH,FW,FC,K}; prm = {sy,sx,pt,pb,pl,pr,dily,dilx}.
 * y = patches * F + 1 * b' per image and filter group (nnconv.cu:105-152);
 * each output is the sum over the filter volume in ascending column order,
 * then the bias is added. */
static int FN(conv_forward)(T* y, T const* x, T const* f, T const* b, int const* shape, int const* prm)
{
  int H = shape[0], W = shape[1], C = shape[2], N = shape[3], FH = shape[4], FW = shape[5], FC = shape[6], K = shape[7];
  int sy = prm[0], sx = prm[1], pt = prm[2], pb = prm[3], pl = prm[4], pr = prm[5], dy = prm[6], dx = prm[7];
  int Ho = (H + pt + pb - ((FH - 1) * dy + 1)) / sy + 1;
  int Wo = (W + pl + pr - ((FW - 1) * dx + 1)) / sx + 1;
  int G = C / FC, Kg = K / G;
  size_t P = (size_t)Ho * Wo, V = (size_t)FH * FW * FC;
  T* patches = (T*)malloc(sizeof(T) * P * V * G);
  T* acc = (T*)malloc(sizeof(T) * P);
  if (!patches || !acc) return 5;
  for (int n = 0; n < N; ++n) {
    FN(im2row)(patches, x + (size_t)H * W * C * n, H, W, C, FH, FW, Ho, Wo, sy, sx, pt, pl, dy, dx);
    for (int k = 0; k < K; ++k) {
      int g = k / Kg;
      T const* pg = patches + P * V * g;
      T const* fk = f + V * k;
      for (size_t p = 0; p < P; ++p) acc[p] = 0;
      for (size_t r = 0; r < V; ++r) {
        T fv = fk[r];
        T const* col = pg + P * r;
        for (size_t p = 0; p < P; ++p) acc[p] += col[p] * fv;
      }
      T* yk = y + P * ((size_t)k + (size_t)K * n);
      if (b) { for (size_t p = 0; p < P; ++p) yk[p] = acc[p] + b[k]; }
      else   { for (size_t p = 0; p < P; ++p) yk[p] = acc[p]; }
    }
  }
  free(patches); free(acc);
  return 0;
}

/* db = sum over images of dy' * 1 (nnconv.cu:229-244);
 * dx_n = row2im(dy_n * F') (nnconv.cu:247-276);
 * df = sum over images of patches_n' * dy_n (nnconv.cu:279-312).
 * Any output may be NULL and is then skipped (nnconv.cu:190-212). */
static int FN(conv_backward)(T* dxo, T* dfo, T* dbo, T const* x, T const* f, T const* dyi,
                             int const* shape, int const* prm)
{
  int H = shape[0], W = shape[1], C = shape[2], N = shape[3], FH = shape[4], FW = shape[5], FC = shape[6], K = shape[7];
  int sy = prm[0], sx = prm[1], pt = prm[2], pb = prm[3], pl = prm[4], pr = prm[5], dy = prm[6], dx = prm[7];
  int Ho = (H + pt + pb - ((FH - 1) * dy + 1)) / sy + 1;
  int Wo = (W + pl + pr - ((FW - 1) * dx + 1)) / sx + 1;
  int G = C / FC, Kg = K / G;
  size_t P = (size_t)Ho * Wo, V = (size_t)FH * FW * FC;
  T* patches = (T*)malloc(sizeof(T) * P * V * G);
  if (!patches) return 5;
  for (int n = 0; n < N; ++n) {
    T const* dyn = dyi + P * K * n;
    if (dbo) {
      for (int k = 0; k < K; ++k) {
        T s = 0;
        for (size_t p = 0; p < P; ++p) s += dyn[P * k + p];
        dbo[k] = (n > 0) ? s + dbo[k] : s;
      }
    }
    if (dxo) {
      for (int g = 0; g < G; ++g)
        for (size_t r = 0; r < V; ++r) {
          T* col = patches + P * (V * g + r);
          for (size_t p = 0; p < P; ++p) col[p] = 0;
          for (int kk = 0; kk < Kg; ++kk) {
            int k = g * Kg + kk;
            T fv = f[V * k + r];
            T const* dyk = dyn + P * k;
            for (size_t p = 0; p < P; ++p) col[p] += dyk[p] * fv;
          }
        }
      FN(row2im)(dxo + (size_t)H * W * C * n, patches, H, W, C, FH, FW, Ho, Wo, sy, sx, pt, pl, dy, dx);
    }
    if (dfo) {
      FN(im2row)(patches, x + (size_t)H * W * C * n, H, W, C, FH, FW, Ho, Wo, sy, sx, pt, pl, dy, dx);
      for (int k = 0; k < K; ++k) {
        int g = k / Kg;
        T const* dyk = dyn + P * k;
        for (size_t r = 0; r < V; ++r) {
          T const* col = patches + P * (V * g + r);
          T s = 0;
          for (size_t p = 0; p < P; ++p) s += col[p] * dyk[p];
          dfo[V * k + r] = (n > 0) ? s + dfo[V * k + r] : s;
        }
      }
    }
  }
  free(patches);
  return 0;
}

/* ------------------------------------------------------------------ */
/* Fully connected (nnfullyconnected.cu:30-102, :108-185)              */
/* ------------------------------------------------------------------ */

/* y(K x N) = F'(K x V) x(V x N) + b 1'. */
static int FN(fc_forward)(T* y, T const* x, T const* f, T const* b, int const* shape)
{
  size_t V = (size_t)shape[0] * shape[1] * shape[2];
  int N = shape[3], K = shape[7];
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) {
      T s = 0;
      for (size_t v = 0; v < V; ++v) s += f[V * k + v] * x[V * n + v];
      y[(size_t)K * n + k] = b ? s + b[k] : s;
    }
  return 0;
}

/* df(V x K) = x(V x N) dy'(N x K); dx(V x N) = F(V x K) dy(K x N); db = dy 1. */
static int FN(fc_backward)(T* dx, T* df, T* db, T const* x, T const* f, T const* dy, int const* shape)
{
  size_t V = (size_t)shape[0] * shape[1] * shape[2];
  int N = shape[3], K = shape[7];
  if (df)
    for (int k = 0; k < K; ++k)
      for (size_t v = 0; v < V; ++v) {
        T s = 0;
        for (int n = 0; n < N; ++n) s += x[V * n + v] * dy[(size_t)K * n + k];
        df[V * k + v] = s;
      }
  if (dx)
    for (int n = 0; n < N; ++n)
      for (size_t v = 0; v < V; ++v) {
        T s = 0;
        for (int k = 0; k < K; ++k) s += f[V * k + v] * dy[(size_t)K * n + k];
        dx[V * n + v] = s;
      }
  if (db)
    for (int k = 0; k < K; ++k) {
      T s = 0;
      for (int n = 0; n < N; ++n) s += dy[(size_t)K * n + k];
      db[k] = s;
    }
  return 0;
}

/* ------------------------------------------------------------------ */
/* Bias (nnbias.cu:37-96, :102-175)                                    */
/* ------------------------------------------------------------------ */

/* With a bias and bmult != 0: y = ymult*y + bmult*b (nnbias.cu:51-76);
 * otherwise y is filled with zeros, whatever ymult is (:78-82).  Then
 * xmult*x is added (:85-91). */
static int FN(bias_forward)(T* y, double ymult, T const* x, double xmult, T const* b, double bmult,
                            int H, int W, int K, int N)
{
  size_t P = (size_t)H * W;
  if (b && bmult != 0) {
    T bm = (T)bmult, ym = (T)ymult;
    for (int n = 0; n < N; ++n)
      for (int k = 0; k < K; ++k) {
        T* yk = y + P * ((size_t)k + (size_t)K * n);
        T v = bm * b[k];
        if (ym == (T)0) { for (size_t p = 0; p < P; ++p) yk[p] = v; }
        else            { for (size_t p = 0; p < P; ++p) yk[p] = v + ym * yk[p]; }
      }
  } else {
    for (size_t i = 0; i < P * K * N; ++i) y[i] = 0;
  }
  if (x && xmult != 0) {
    T xm = (T)xmult;
    for (size_t i = 0; i < P * K * N; ++i) y[i] += xm * x[i];
  }
  return 0;
}

/* db = dbmult*db + bmult * sum_{h,w,n} dy (nnbias.cu:127-149);
 * dx = dxmult*dx + xmult*dy (:152-170; the zero-fill branch at :155 is never
 * taken for a non-null tensor, so a zero multiplier still scales). */
static int FN(bias_backward)(T* dx, double dxmult, T* db, double dbmult, double xmult, double bmult,
                             T const* dy, int H, int W, int K, int N)
{
  size_t P = (size_t)H * W;
  if (db) {
    for (int n = 0; n < N; ++n)
      for (int k = 0; k < K; ++k) {
        T s = 0;
        T const* dyk = dy + P * ((size_t)k + (size_t)K * n);
        for (size_t p = 0; p < P; ++p) s += dyk[p];
        T beta = (n == 0) ? (T)dbmult : (T)1;
        db[k] = (beta == (T)0) ? (T)bmult * s : (T)bmult * s + beta * db[k];
      }
  }
  if (dx) {
    size_t n = P * K * N;
    if (dxmult != 1.0) { T m = (T)dxmult; for (size_t i = 0; i < n; ++i) dx[i] = m * dx[i]; }
    T xm = (T)xmult;
    for (size_t i = 0; i < n; ++i) dx[i] += xm * dy[i];
  }
  return 0;
}

/* Convolution transpose (nnconv.cu:323-421).  shape = {H,W,C,N,FH,FW,FD,FN} (FN == C); prm = {upY,upX,cropT,cropB,
 * cropL,cropR,numGroups}.  The convolution it re-uses has the transposed convolution's output as its input, stride =
 * upsample and pad = crop.  Forward: that convolution's data gradient, image by image (:338-367), then the bias
 * (:368-370).  Backward: dx = its forward pass of dy (:398-403), df = its filter gradient with data and output
 * derivative exchanged (:405-409), db = sum of dy (:411-414). */
static void FN(convt_geom)(int const* shape, int const* prm, int* cshape, int* cprm)
{
  int H = shape[0], W = shape[1], FH = shape[4], FW = shape[5], FD = shape[6], G = prm[6];
  cshape[0] = (H - 1) * prm[0] - (prm[2] + prm[3]) + FH;
  cshape[1] = (W - 1) * prm[1] - (prm[4] + prm[5]) + FW;
  cshape[2] = FD * G; cshape[3] = shape[3];
  cshape[4] = FH; cshape[5] = FW; cshape[6] = FD; cshape[7] = shape[2];
  cprm[0] = prm[0]; cprm[1] = prm[1]; cprm[2] = prm[2]; cprm[3] = prm[3]; cprm[4] = prm[4]; cprm[5] = prm[5];
  cprm[6] = 1; cprm[7] = 1;
}

static int FN(convt_forward)(T* y, T const* x, T const* f, T const* b, int const* shape, int const* prm)
{
  int cs[8], cp[8];
  FN(convt_geom)(shape, prm, cs, cp);
  int N = shape[3];
  size_t inStep = (size_t)shape[0] * shape[1] * shape[2], outStep = (size_t)cs[0] * cs[1] * cs[2];
  cs[3] = 1;
  for (int n = 0; n < N; ++n) {
    int rc = FN(conv_backward)(y + outStep * n, NULL, NULL, NULL, f, x + inStep * n, cs, cp);
    if (rc) return rc;
  }
  if (b) return FN(bias_forward)(y, 1.0, NULL, 0.0, b, 1.0, cs[0], cs[1], cs[2], N);
  return 0;
}

static int FN(convt_backward)(T* dx, T* df, T* db, T const* x, T const* f, T const* dy, int const* shape, int const* prm)
{
  int cs[8], cp[8], rc = 0;
  FN(convt_geom)(shape, prm, cs, cp);
  if (dx) { rc = FN(conv_forward)(dx, dy, f, NULL, cs, cp); if (rc) return rc; }
  if (df) { rc = FN(conv_backward)(NULL, df, NULL, dy, NULL, x, cs, cp); if (rc) return rc; }
  if (db) rc = FN(bias_backward)(NULL, 0.0, db, 0.0, 0.0, 1.0, dy, cs[0], cs[1], cs[2], cs[3]);
  return rc;
}

/* ------------------------------------------------------------------ */
/* Batch normalisation (nnbnorm.cu:46-164 helpers, :170-365 functors)  */
/* ------------------------------------------------------------------ */

/* Serial accumulation in T over images then pixels, per channel (nnbnorm.cu:53-70). */
static void FN(bn_moments)(T* mom, T const* x, int WH, int C, int N, T eps)
{
  int mass = WH * N;
  for (int c = 0; c < C; ++c) {
    T s = 0, q = 0;
    for (int n = 0; n < N; ++n)
      for (int i = 0; i < WH; ++i) {
        T v = x[(size_t)i + (size_t)WH * ((size_t)c + (size_t)C * n)];
        s += v; q += v * v;
      }
    T mean = s / mass;
    T s2 = q / mass - mean * mean;
    if (!(s2 > (T)0)) s2 = (T)0;          /* std::max((T)0, s2), :67 */
    mom[c] = mean;
    mom[c + C] = (T)sqrt(s2 + eps);
  }
}

/* y = g/sigma * (x - mean) + b (nnbnorm.cu:192-203). */
static int FN(bnorm_forward_moment)(T* y, T const* mom, T const* x, T const* g, T const* b,
                                    int H, int W, int C, int N, double eps)
{
  (void)eps;
  int WH = H * W;
  for (int c = 0; c < C; ++c) {
    T mean = mom[c], sigma = mom[c + C], coef = g[c] / sigma, bias = b[c];
    for (int n = 0; n < N; ++n)
      for (int i = 0; i < WH; ++i) {
        size_t o = (size_t)i + (size_t)WH * ((size_t)c + (size_t)C * n);
        y[o] = coef * (x[o] - mean) + bias;
      }
  }
  return 0;
}

static int FN(bnorm_forward)(T* y, T* mom, T const* x, T const* g, T const* b, int H, int W, int C, int N, double eps)
{
  T* own = mom ? mom : (T*)malloc(sizeof(T) * 2 * C);
  if (!own) return 5;
  FN(bn_moments)(own, x, H * W, C, N, (T)eps);
  FN(bnorm_forward_moment)(y, own, x, g, b, H, W, C, N, eps);
  if (!mom) free(own);
  return 0;
}

/* dx = G1*(dy - db/m) - G2*(x - mean), G1 = g/sigma, G2 = G1*dg/(m*sigma)
 * (nnbnorm.cu:136-164). */
static void FN(bn_dx)(T* dx, T const* mom, T const* x, T const* g, T const* dg, T const* db, T const* dy,
                      int WH, int C, int N)
{
  T mass = (T)(WH * N);
  for (int c = 0; c < C; ++c) {
    T mean = mom[c], sigma = mom[c + C];
    T muz = db[c] / mass;
    T G1 = g[c] / sigma;
    T G2 = G1 * dg[c] / (mass * sigma);
    for (int n = 0; n < N; ++n)
      for (int i = 0; i < WH; ++i) {
        size_t o = (size_t)i + (size_t)WH * ((size_t)c + (size_t)C * n);
        dx[o] = G1 * (dy[o] - muz) - G2 * (x[o] - mean);
      }
  }
}

/* Moments given: dg = (sum dy*x - mean*sum dy)/sigma, db = sum dy (nnbnorm.cu:75-100). */
static int FN(bnorm_backward_moment)(T* dx, T* dg, T* db, T const* mom, T const* x, T const* g, T const* b,
                                     T const* dy, int H, int W, int C, int N, double eps)
{
  (void)b; (void)eps;
  int WH = H * W;
  for (int c = 0; c < C; ++c) {
    T sxy = 0, sy = 0;
    for (int n = 0; n < N; ++n)
      for (int i = 0; i < WH; ++i) {
        size_t o = (size_t)i + (size_t)WH * ((size_t)c + (size_t)C * n);
        sxy += dy[o] * x[o]; sy += dy[o];
      }
    db[c] = sy;
    dg[c] = (sxy - mom[c] * sy) / mom[c + C];
  }
  FN(bn_dx)(dx, mom, x, g, dg, db, dy, WH, C, N);
  return 0;
}

/* Moments computed in the same sweep (nnbnorm.cu:102-134); written to mom when non-NULL. */
static int FN(bnorm_backward)(T* dx, T* dg, T* db, T* mom, T const* x, T const* g, T const* b, T const* dy,
                              int H, int W, int C, int N, double eps)
{
  (void)b;
  int WH = H * W;
  T* own = mom ? mom : (T*)malloc(sizeof(T) * 2 * C);
  if (!own) return 5;
  T mass = (T)(WH * N);
  for (int c = 0; c < C; ++c) {
    T s = 0, q = 0, sxy = 0, sy = 0;
    for (int n = 0; n < N; ++n)
      for (int i = 0; i < WH; ++i) {
        size_t o = (size_t)i + (size_t)WH * ((size_t)c + (size_t)C * n);
        s += x[o]; q += x[o] * x[o]; sxy += dy[o] * x[o]; sy += dy[o];
      }
    T mean = s / mass;
    T s2 = q / mass - mean * mean;
    if (!(s2 > (T)0)) s2 = (T)0;
    T sigma = (T)sqrt(s2 + (T)eps);
    own[c] = mean; own[c + C] = sigma;
    db[c] = sy;
    dg[c] = (sxy - mean * sy) / sigma;
  }
  FN(bn_dx)(dx, own, x, g, dg, db, dy, WH, C, N);
  if (!mom) free(own);
  return 0;
}

/* ------------------------------------------------------------------ */
/* Pooling (nnpooling.cu:102-142 forward, :170-214 backward)           */
/* ------------------------------------------------------------------ */

/* prm = {poolH,poolW,sy,sx,pt,pb,pl,pr,method}.  Windows are clipped to the
 * image; max starts from -inf; average divides by the CLIPPED window area
 * (nnpooling.cu:71-75,128). */
static int FN(pool_forward)(T* y, T const* x, int H, int W, int C, int N, int const* prm)
{
  int ph = prm[0], pw = prm[1], sy = prm[2], sx = prm[3], pt = prm[4], pb = prm[5], pl = prm[6], pr = prm[7];
  int Ho = (H + pt + pb - ph) / sy + 1, Wo = (W + pl + pr - pw) / sx + 1;
  for (size_t z = 0; z < (size_t)C * N; ++z) {
    T const* xz = x + (size_t)H * W * z;
    T* yz = y + (size_t)Ho * Wo * z;
    for (int wo = 0; wo < Wo; ++wo)
      for (int ho = 0; ho < Ho; ++ho) {
        int x1 = wo * sx - pl, y1 = ho * sy - pt;
        int x2 = x1 + pw < W ? x1 + pw : W, y2 = y1 + ph < H ? y1 + ph : H;
        if (x1 < 0) x1 = 0;
        if (y1 < 0) y1 = 0;
        if (prm[8] == 0) {
          T best = -(T)INFINITY;
          for (int u = x1; u < x2; ++u)
            for (int v = y1; v < y2; ++v) { T t = xz[(size_t)u * H + v]; best = (best < t) ? t : best; }
          yz[(size_t)wo * Ho + ho] = best;
        } else {
          T s = 0, scale = (T)1 / (T)((y2 - y1) * (x2 - x1));
          for (int u = x1; u < x2; ++u)
            for (int v = y1; v < y2; ++v) s += xz[(size_t)u * H + v];
          yz[(size_t)wo * Ho + ho] = s * scale;
        }
      }
  }
  return 0;
}

/* dx starts at zero (the gateway zero-fills it, vl_nnpool.cu:255-259) and is
 * accumulated into, windows visited wo-outer / ho-inner.  Max: scan u (width)
 * outer, v (height) inner; the first element strictly greater than the running
 * best (initially -inf) wins; no winner => nothing is routed
 * (nnpooling.cu:47-61). */
static int FN(pool_backward)(T* dx, T const* x, T const* dy, int H, int W, int C, int N, int const* prm)
{
  int ph = prm[0], pw = prm[1], sy = prm[2], sx = prm[3], pt = prm[4], pb = prm[5], pl = prm[6], pr = prm[7];
  int Ho = (H + pt + pb - ph) / sy + 1, Wo = (W + pl + pr - pw) / sx + 1;
  memset(dx, 0, sizeof(T) * (size_t)H * W * C * N);
  for (size_t z = 0; z < (size_t)C * N; ++z) {
    T const* xz = x + (size_t)H * W * z;
    T* dxz = dx + (size_t)H * W * z;
    T const* dyz = dy + (size_t)Ho * Wo * z;
    for (int wo = 0; wo < Wo; ++wo)
      for (int ho = 0; ho < Ho; ++ho) {
        int x1 = wo * sx - pl, y1 = ho * sy - pt;
        int x2 = x1 + pw < W ? x1 + pw : W, y2 = y1 + ph < H ? y1 + ph : H;
        if (x1 < 0) x1 = 0;
        if (y1 < 0) y1 = 0;
        T d = dyz[(size_t)wo * Ho + ho];
        if (prm[8] == 0) {
          T best = -(T)INFINITY;
          long where = -1;
          for (int u = x1; u < x2; ++u)
            for (int v = y1; v < y2; ++v) {
              T t = xz[(size_t)u * H + v];
              if (t > best) { best = t; where = (long)u * H + v; }
            }
          if (where >= 0) dxz[where] += d;
        } else {
          T scale = (T)1 / (T)((y2 - y1) * (x2 - x1));
          for (int u = x1; u < x2; ++u)
            for (int v = y1; v < y2; ++v) dxz[(size_t)u * H + v] += d * scale;
        }
      }
  }
  return 0;
}

/* ------------------------------------------------------------------ */
/* ROI pooling (nnroipooling.cu:102-189 forward, :217-305 backward)    */
/* ------------------------------------------------------------------ */

typedef struct { int image, start_h, start_w; T bin_h, bin_w; } FN(roi_t);

/* ROI geometry (nnroipooling.cu:120-148).  The affine map is evaluated in
 * double (transform is double) and stored to T; rounding is C round() (half
 * away from zero); the image index is clamped to [1,N]; the bin size is the
 * double quotient stored to T. */
static FN(roi_t) FN(roi_geom)(T const* r, double const* tf, int N, int S0, int S1)
{
  FN(roi_t) g;
  T u1_ = r[1], v1_ = r[2], u2_ = r[3], v2_ = r[4];
  T u1 = (T)(tf[0] * u1_ + tf[2] * v1_ + tf[4]);
  T v1 = (T)(tf[1] * u1_ + tf[3] * v1_ + tf[5]);
  T u2 = (T)(tf[0] * u2_ + tf[2] * v2_ + tf[4]);
  T v2 = (T)(tf[1] * u2_ + tf[3] * v2_ + tf[5]);
  int image = (int)r[0];
  g.start_h = (int)round(v1) - 1;
  g.start_w = (int)round(u1) - 1;
  int end_h = (int)round(v2) - 1, end_w = (int)round(u2) - 1;
  int rh = end_h - g.start_h + 1, rw = end_w - g.start_w + 1;
  if (rh < 1) rh = 1;
  if (rw < 1) rw = 1;
  image -= 1;
  if (image < 0) image = 0;
  if (image > N - 1) image = N - 1;
  g.image = image;
  g.bin_h = (T)((double)rh / S0);
  g.bin_w = (T)((double)rw / S1);
  return g;
}

static int FN(clampi)(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* Bin bounds (nnroipooling.cu:155-165): floor/ceil of the T product, shifted
 * by the ROI start, clamped to [0, extent]. */
static void FN(roi_bin)(int p, T bin, int start, int extent, int* lo, int* hi)
{
  int a = (int)floor(((T)p) * bin);
  int b = (int)ceil(((T)(p + 1)) * bin);
  *lo = FN(clampi)(a + start, 0, extent);
  *hi = FN(clampi)(b + start, 0, extent);
}

/* Writes bin bounds {hstart,hend,wstart,wend} for every (roi, ph, pw):
 * bounds[4*(ph + S0*(pw + S1*roi)) + i].  Used to check the device's bin
 * arithmetic bit for bit. */
static int FN(roipool_bounds)(int* bounds, int* images, T const* rois, int H, int W, int N, int numROIs,
                              int S0, int S1, double const* tf)
{
  for (int r = 0; r < numROIs; ++r) {
    FN(roi_t) g = FN(roi_geom)(rois + 5 * (size_t)r, tf, N, S0, S1);
    if (images) images[r] = g.image;
    for (int pw = 0; pw < S1; ++pw) {
      int ws, we;
      FN(roi_bin)(pw, g.bin_w, g.start_w, W, &ws, &we);
      for (int ph = 0; ph < S0; ++ph) {
        int hs, he;
        FN(roi_bin)(ph, g.bin_h, g.start_h, H, &hs, &he);
        int* o = bounds + 4 * ((size_t)ph + (size_t)S0 * ((size_t)pw + (size_t)S1 * r));
        o[0] = hs; o[1] = he; o[2] = ws; o[3] = we;
      }
    }
  }
  return 0;
}

/* Output S0 x S1 x C x K written roi -> channel -> pw -> ph; empty bin => 0. */
static int FN(roipool_forward)(T* y, T const* x, T const* rois, int H, int W, int C, int N, int numROIs,
                               int S0, int S1, double const* tf, int method)
{
  for (int r = 0; r < numROIs; ++r) {
    FN(roi_t) g = FN(roi_geom)(rois + 5 * (size_t)r, tf, N, S0, S1);
    for (int c = 0; c < C; ++c) {
      T const* xz = x + (size_t)H * W * ((size_t)c + (size_t)C * g.image);
      for (int pw = 0; pw < S1; ++pw) {
        int ws, we;
        FN(roi_bin)(pw, g.bin_w, g.start_w, W, &ws, &we);
        for (int ph = 0; ph < S0; ++ph) {
          int hs, he;
          FN(roi_bin)(ph, g.bin_h, g.start_h, H, &hs, &he);
          T out = 0;
          if (he > hs && we > ws) {
            if (method == 0) {
              T best = -(T)INFINITY;
              for (int w = ws; w < we; ++w)
                for (int h = hs; h < he; ++h) { T t = xz[(size_t)w * H + h]; best = (best < t) ? t : best; }
              out = best;
            } else {
              T s = 0;
              for (int w = ws; w < we; ++w)
                for (int h = hs; h < he; ++h) s += xz[(size_t)w * H + h];
              out = s * ((T)1 / (T)((he - hs) * (we - ws)));
            }
          }
          *y++ = out;
        }
      }
    }
  }
  return 0;
}

/* dx zeroed first (nnroipooling.cu:237), then per bin: max routes dy to the
 * first strictly-greater element in w-outer / h-inner order (:288-295); average
 * adds dy/area to every pixel of the bin. */
static int FN(roipool_backward)(T* dx, T const* x, T const* rois, T const* dy, int H, int W, int C, int N,
                                int numROIs, int S0, int S1, double const* tf, int method)
{
  memset(dx, 0, sizeof(T) * (size_t)H * W * C * N);
  for (int r = 0; r < numROIs; ++r) {
    FN(roi_t) g = FN(roi_geom)(rois + 5 * (size_t)r, tf, N, S0, S1);
    for (int c = 0; c < C; ++c) {
      size_t off = (size_t)H * W * ((size_t)c + (size_t)C * g.image);
      T const* xz = x + off;
      T* dxz = dx + off;
      for (int pw = 0; pw < S1; ++pw) {
        int ws, we;
        FN(roi_bin)(pw, g.bin_w, g.start_w, W, &ws, &we);
        for (int ph = 0; ph < S0; ++ph) {
          int hs, he;
          FN(roi_bin)(ph, g.bin_h, g.start_h, H, &hs, &he);
          T d = *dy++;
          if (method == 0) {
            T best = -(T)INFINITY;
            long where = -1;
            for (int w = ws; w < we; ++w)
              for (int h = hs; h < he; ++h) {
                T t = xz[(size_t)w * H + h];
                if (t > best) { best = t; where = (long)w * H + h; }
              }
            if (where >= 0) dxz[where] += d;
          } else {
            T scale = (T)1 / (T)((he - hs) * (we - ws));
            for (int w = ws; w < we; ++w)
              for (int h = hs; h < he; ++h) dxz[(size_t)w * H + h] += d * scale;
          }
        }
      }
    }
  }
  return 0;
}

/* ------------------------------------------------------------------ */
/* Bilinear sampler (nnbilinearsampler.cu:32-149)                      */
/* ------------------------------------------------------------------ */

/* Grid entries are (gy, gx) in [-1,1], y first (:76-77).  p = 0.5*(g+1)*(extent-1);
 * s = floor(p).  The reference guards the taps with `-1 <= sy && sy < inHeight`
 * where inHeight is size_t (:92), so sy is converted to unsigned for the second
 * test and sy == -1 (likewise sx == -1) FAILS it: a sample whose floor is -1
 * contributes nothing at all.  That behaviour is reproduced here. */
#define SAMPLER_COMMON                                                            \
  T py = grid[2 * q], px = grid[2 * q + 1];                                       \
  py = (T)0.5 * (py + (T)1.0) * (T)(H - 1);                                       \
  px = (T)0.5 * (px + (T)1.0) * (T)(W - 1);                                       \
  int sx = (int)floor(px), sy = (int)floor(py);                                   \
  int inside = (sy >= 0 && sy < H && sx >= 0 && sx < W);                          \
  T wx = px - (T)sx, wy = py - (T)sy;

static int FN(sampler_forward)(T* y, T const* x, T const* grid_all, int H, int W, int C, int N,
                               int Ho, int Wo, int Ng)
{
  int group = Ng / N;
  size_t Q = (size_t)Ho * Wo;
  for (int n = 0; n < Ng; ++n) {
    T const* grid = grid_all + 2 * Q * n;
    for (int c = 0; c < C; ++c) {
      T const* xz = x + (size_t)H * W * ((size_t)c + (size_t)C * (n / group));
      T* yz = y + Q * ((size_t)c + (size_t)C * n);
      for (size_t q = 0; q < Q; ++q) {
        SAMPLER_COMMON
        T acc = 0;
        if (inside)
          for (int j = 0; j < 2; ++j)
            for (int i = 0; i < 2; ++i) {
              int ssy = sy + i, ssx = sx + j;
              if (ssy < 0 || ssy >= H || ssx < 0 || ssx >= W) continue;
              T wwx = (T)(1 - j) * ((T)1 - wx) + (T)j * wx;
              T wwy = (T)(1 - i) * ((T)1 - wy) + (T)i * wy;
              acc += (wwx * wwy) * xz[ssy + (size_t)ssx * H];
            }
        yz[q] = acc;
      }
    }
  }
  return 0;
}

/* dx[tap] += ww*dy (:115); dgrid_y += 0.5*(H-1) * sum_taps (2i-1)*wwx*dy*x,
 * dgrid_x likewise with (2j-1)*wwy (:117-131), accumulated over channels.
 * Both outputs start from zero (vl_nnbilinearsampler.cu:176-181). */
static int FN(sampler_backward)(T* dx, T* dgrid_all, T const* x, T const* grid_all, T const* dy,
                                int H, int W, int C, int N, int Ho, int Wo, int Ng)
{
  int group = Ng / N;
  size_t Q = (size_t)Ho * Wo;
  if (dx) memset(dx, 0, sizeof(T) * (size_t)H * W * C * N);
  if (dgrid_all) memset(dgrid_all, 0, sizeof(T) * 2 * Q * Ng);
  for (int n = 0; n < Ng; ++n) {
    T const* grid = grid_all + 2 * Q * n;
    T* dgrid = dgrid_all ? dgrid_all + 2 * Q * n : NULL;
    for (int c = 0; c < C; ++c) {
      size_t off = (size_t)H * W * ((size_t)c + (size_t)C * (n / group));
      T const* xz = x + off;
      T* dxz = dx ? dx + off : NULL;
      T const* dyz = dy + Q * ((size_t)c + (size_t)C * n);
      for (size_t q = 0; q < Q; ++q) {
        SAMPLER_COMMON
        T d = dyz[q], dgx = 0, dgy = 0;
        if (inside)
          for (int j = 0; j < 2; ++j)
            for (int i = 0; i < 2; ++i) {
              int ssy = sy + i, ssx = sx + j;
              if (ssy < 0 || ssy >= H || ssx < 0 || ssx >= W) continue;
              T wwx = (T)(1 - j) * ((T)1 - wx) + (T)j * wx;
              T wwy = (T)(1 - i) * ((T)1 - wy) + (T)i * wy;
              if (dxz) dxz[ssy + (size_t)ssx * H] += (wwx * wwy) * d;
              if (dgrid) {
                T xv = xz[ssy + (size_t)ssx * H];
                dgx += (T)(2 * j - 1) * wwy * d * xv;
                dgy += (T)(2 * i - 1) * wwx * d * xv;
              }
            }
        if (dgrid) {
          dgrid[2 * q] += (T)0.5 * (T)(H - 1) * dgy;
          dgrid[2 * q + 1] += (T)0.5 * (T)(W - 1) * dgx;
        }
      }
    }
  }
  return 0;
}
#undef SAMPLER_COMMON

/* ------------------------------------------------------------------ */
/* Glue blocks that exist only as MATLAB in the reference              */
/* ------------------------------------------------------------------ */

/* matlab/vl_nnrelu.m:43-48 with leak 0: y = max(x,0); dx = dy .* (x > 0). */
static int FN(relu_forward)(T* y, T const* x, size_t n)
{ for (size_t i = 0; i < n; ++i) y[i] = x[i] > (T)0 ? x[i] : (T)0; return 0; }
static int FN(relu_backward)(T* dx, T const* x, T const* dy, size_t n)
{ for (size_t i = 0; i < n; ++i) dx[i] = x[i] > (T)0 ? dy[i] : (T)0; return 0; }

/* matlab/vl_nnsoftmaxloss.m:56-84.  x is H x W x C x N, labels c is one class
 * (1-based) per image, broadcast over pixels (:45-52); class 0 skips the image:
 * mass = (c > 0), index max(c - 1, 0) (:55-67).  Forward returns the
 * scalar sum over pixels and images of (xmax + log sum exp(x - xmax) - x_c),
 * divided by N (:72-77,:84).  Backward: dx = dzdy/N * (softmax - onehot). */
static int FN(softmaxloss_forward)(T* loss, T const* x, T const* labels, int H, int W, int C, int N)
{
  size_t P = (size_t)H * W;
  T total = 0;
  for (int n = 0; n < N; ++n)
    for (size_t p = 0; p < P; ++p) {
      T const* xp = x + p + P * (size_t)C * n;
      T xmax = xp[0];
      for (int c = 1; c < C; ++c) if (xp[P * c] > xmax) xmax = xp[P * c];
      T se = 0;
      for (int c = 0; c < C; ++c) se += (T)exp(xp[P * c] - xmax);
      T mass = labels[n] > (T)0 ? (T)1 : (T)0;
      int lab = (int)labels[n] - 1;
      if (lab < 0) lab = 0;
      if (lab >= C) return 1;      /* an indexing error in the reference */
      total += mass * (xmax + (T)log(se) - xp[P * lab]);
    }
  *loss = total / (T)N;
  return 0;
}

static int FN(softmaxloss_backward)(T* dx, T const* x, T const* labels, T dzdy, int H, int W, int C, int N)
{
  size_t P = (size_t)H * W;
  T scale = dzdy / (T)N;
  for (int n = 0; n < N; ++n)
    for (size_t p = 0; p < P; ++p) {
      T const* xp = x + p + P * (size_t)C * n;
      T* dp = dx + p + P * (size_t)C * n;
      T xmax = xp[0];
      for (int c = 1; c < C; ++c) if (xp[P * c] > xmax) xmax = xp[P * c];
      T se = 0;
      for (int c = 0; c < C; ++c) se += (T)exp(xp[P * c] - xmax);
      T mass = labels[n] > (T)0 ? (T)1 : (T)0;
      int lab = (int)labels[n] - 1;
      if (lab < 0) lab = 0;
      if (lab >= C) return 1;      /* an indexing error in the reference */
      for (int c = 0; c < C; ++c) {
        T v = (T)exp(xp[P * c] - xmax) / se;
        if (c == lab) v -= (T)1;
        dp[P * c] = v * (mass * scale);
      }
    }
  return 0;
}

/* vl::nn::LRN (bits/nnnormalize.cu:143-226 forward, :232-400 backward): y_t = x_t * L_t^-beta,
 * L_t = kappa + alpha * sum of x_q^2 over q in [t - m1, t + m2] clipped to the channels, m1 = (N - 1) / 2,
 * m2 = N - m1 - 1; the window sum slides (acc += ap^2 - am^2, :169-176).  Backward as the plain loop nest of the
 * reference (:257-288): dx_t += dz_t * L_t^-beta and dx_q -= dz_t * x_t * x_q * 2*alpha*beta * L_t^(-beta-1) for the q in
 * t's window.  The reference's compiled CPU code replaces pow by a cubic approximation of log2 and exp2 (:49-125); this
 * restatement uses the C library's pow, so it agrees with the compiled code only to that approximation's error. */
static int FN(lrn_forward)(T* y, T const* x, int H, int W, int C, int N, int depth, double kappa, double alpha, double beta)
{
  size_t P = (size_t)H * W;
  int m1 = (depth - 1) / 2, m2 = depth - m1 - 1;
  for (int n = 0; n < N; ++n)
    for (size_t p = 0; p < P; ++p) {
      T const* xp = x + p + P * (size_t)C * n;
      T* yp = y + p + P * (size_t)C * n;
      T acc = 0;
      for (int t = -m2; t < C; ++t) {
        T ap = 0, am = 0;
        if (t - m1 - 1 >= 0) am = xp[P * (t - m1 - 1)];
        if (t + m2 < C) ap = xp[P * (t + m2)];
        acc += ap * ap - am * am;
        if (t >= 0) yp[P * t] = xp[P * t] * (T)pow((double)((T)kappa + (T)alpha * acc), -beta);
      }
    }
  return 0;
}

static int FN(lrn_backward)(T* dx, T const* x, T const* dz, int H, int W, int C, int N, int depth, double kappa,
                            double alpha, double beta)
{
  size_t P = (size_t)H * W;
  int m1 = (depth - 1) / 2, m2 = depth - m1 - 1;
  T ab2 = (T)(2 * alpha * beta);
  for (int n = 0; n < N; ++n)
    for (size_t p = 0; p < P; ++p) {
      T const* xp = x + p + P * (size_t)C * n;
      T const* zp = dz + p + P * (size_t)C * n;
      T* yp = dx + p + P * (size_t)C * n;
      T acc = 0;
      for (int t = 0; t < C; ++t) yp[P * t] = 0;
      for (int t = -m2; t < C; ++t) {
        int q1 = t - m1, q2 = t + m2;
        T ap = 0, am = 0;
        if (t - m1 - 1 >= 0) am = xp[P * (t - m1 - 1)]; else q1 = 0;
        if (t + m2 < C) ap = xp[P * (t + m2)]; else q2 = C - 1;
        acc += ap * ap - am * am;
        T L = (T)kappa + (T)alpha * acc;
        T Lbeta = (T)pow((double)L, -beta);
        T Lbeta1 = Lbeta / L;
        if (t >= 0) {
          yp[P * t] += zp[P * t] * Lbeta;
          for (int q = q1; q <= q2; ++q) yp[P * q] -= zp[P * t] * xp[P * t] * xp[P * q] * ab2 * Lbeta1;
        }
      }
    }
  return 0;
}

/* matlab/vl_nnsoftmax.m: E = exp(x - max over channels); Y = E / sum(E); backward Y .* (dzdY - sum(dzdY .* Y)). */
static int FN(softmax)(T* out, T const* x, T const* dz, int H, int W, int C, int N)
{
  size_t P = (size_t)H * W;
  for (int n = 0; n < N; ++n)
    for (size_t p = 0; p < P; ++p) {
      T const* xp = x + p + P * (size_t)C * n;
      T* op = out + p + P * (size_t)C * n;
      T xmax = xp[0], se = 0, dot = 0;
      for (int c = 1; c < C; ++c) if (xp[P * c] > xmax) xmax = xp[P * c];
      for (int c = 0; c < C; ++c) se += (T)exp(xp[P * c] - xmax);
      if (dz) for (int c = 0; c < C; ++c) dot += dz[p + P * (size_t)C * n + P * c] * ((T)exp(xp[P * c] - xmax) / se);
      for (int c = 0; c < C; ++c) {
        T yv = (T)exp(xp[P * c] - xmax) / se;
        op[P * c] = dz ? yv * (dz[p + P * (size_t)C * n + P * c] - dot) : yv;
      }
    }
  return 0;
}

#undef IDX4
