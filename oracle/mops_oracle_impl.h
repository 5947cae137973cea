/* Test infrastructure, not product code: a plain-C restatement of the CPU algorithms of
 * lab-cosmo/mops, included once per scalar type by mops_oracle.c (T = scalar type,
 * FN(name) = name with the type suffix). Every function states the reference lines it
 * follows. Sums are taken in the reference's order for each output element (entries,
 * monomials and triplets in ascending input order), so results agree with the reference
 * CPU library to rounding of the last few bits, not merely to tolerance.
 *
 * Conventions shared by all functions: row-major contiguous arrays, int32 zero-based
 * indices, outputs fully overwritten, a NULL gradient output means "skip it".
 * Index ranges are the caller's business (the tests feed valid indices). */

/* O[i] = sum_j C[j] * prod_k A[i, P[j,k]]        mops/src/hpe/cpu.tpp:42-58 */
void FN(oracle_hpe)(T *O, const T *A, const T *C, const int32_t *P,
                    int64_t I, int64_t N, int64_t J, int64_t K) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < I; i++) {
        const T *a = A + i * N;
        T acc = 0;
        for (int64_t j = 0; j < J; j++) {
            T t = C[j];
            for (int64_t k = 0; k < K; k++) t *= a[P[j * K + k]];
            acc += t;
        }
        O[i] = acc;
    }
}

/* gA[i, P[j,k]] += gO[i]*C[j] * prod_{l != k} A[i, P[j,l]]   mops/src/hpe/cpu.tpp:174-189 */
void FN(oracle_hpe_vjp)(T *gA, const T *gO, const T *A, const T *C, const int32_t *P,
                        int64_t I, int64_t N, int64_t J, int64_t K) {
    if (!gA) return;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < I; i++) {
        const T *a = A + i * N;
        T *g = gA + i * N;
        for (int64_t n = 0; n < N; n++) g[n] = 0;
        for (int64_t j = 0; j < J; j++) {
            T base = C[j] * gO[i];
            for (int64_t k = 0; k < K; k++) {
                T t = base;
                for (int64_t l = 0; l < K; l++)
                    if (l != k) t *= a[P[j * K + l]];
                g[P[j * K + k]] += t;
            }
        }
    }
}

/* Second-order terms of HPE.  mops/src/hpe/cpu.tpp:275-539,
 * python/mops/src/mops/reference_implementations.py:322-376
 *   ggO[i]          += C[j] ggA[i,P[j,k]] prod_{l != k} A[i,P[j,l]]                  (all j, k)
 *   gA2[i, P[j,l]]  += gO[i] C[j] ggA[i,P[j,k]] prod_{m != k, m != l} A[i,P[j,m]]    (all j, l, k != l)
 * ggA may be NULL (both terms vanish); each output may be NULL (skipped). */
void FN(oracle_hpe_vjp_vjp)(T *ggO, T *gA2, const T *ggA, const T *gO, const T *A, const T *C,
                            const int32_t *P, int64_t I, int64_t N, int64_t J, int64_t K) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < I; i++) {
        const T *a = A + i * N;
        if (ggO) ggO[i] = 0;
        if (gA2) for (int64_t n = 0; n < N; n++) gA2[i * N + n] = 0;
        if (!ggA) continue;
        const T *h = ggA + i * N;
        for (int64_t j = 0; j < J; j++) {
            const int32_t *p = P + j * K;
            if (ggO)
                for (int64_t k = 0; k < K; k++) {
                    T t = C[j] * h[p[k]];
                    for (int64_t l = 0; l < K; l++)
                        if (l != k) t *= a[p[l]];
                    ggO[i] += t;
                }
            if (gA2)
                for (int64_t l = 0; l < K; l++)
                    for (int64_t k = 0; k < K; k++) {
                        if (k == l) continue;
                        T t = C[j] * gO[i] * h[p[k]];
                        for (int64_t m = 0; m < K; m++)
                            if (m != k && m != l) t *= a[p[m]];
                        gA2[i * N + p[l]] += t;
                    }
        }
    }
}

/* O[i, PO[k]] += C[k]*A[i,PA[k]]*B[i,PB[k]]      mops/src/sap/cpu.tpp:65-78 */
void FN(oracle_sap)(T *O, const T *A, const T *B, const T *C, const int32_t *PA,
                    const int32_t *PB, const int32_t *PO, int64_t I, int64_t nA, int64_t nB,
                    int64_t nO, int64_t K) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < I; i++) {
        T *o = O + i * nO;
        for (int64_t n = 0; n < nO; n++) o[n] = 0;
        for (int64_t k = 0; k < K; k++)
            o[PO[k]] += C[k] * A[i * nA + PA[k]] * B[i * nB + PB[k]];
    }
}

/* gA[i,PA[k]] += gO[i,PO[k]]*C[k]*B[i,PB[k]]; gB symmetric   mops/src/sap/cpu.tpp:197-218 */
void FN(oracle_sap_vjp)(T *gA, T *gB, const T *gO, const T *A, const T *B, const T *C,
                        const int32_t *PA, const int32_t *PB, const int32_t *PO, int64_t I,
                        int64_t nA, int64_t nB, int64_t nO, int64_t K) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < I; i++) {
        if (gA) for (int64_t n = 0; n < nA; n++) gA[i * nA + n] = 0;
        if (gB) for (int64_t n = 0; n < nB; n++) gB[i * nB + n] = 0;
        for (int64_t k = 0; k < K; k++) {
            T go = gO[i * nO + PO[k]];
            if (gA) gA[i * nA + PA[k]] += go * C[k] * B[i * nB + PB[k]];
            if (gB) gB[i * nB + PB[k]] += go * C[k] * A[i * nA + PA[k]];
        }
    }
}

/* Second-order terms of SAP.  python/mops/src/mops/reference_implementations.py:442-509
 *   ggO[i,PO_k] += C_k (ggA[i,PA_k] B[i,PB_k] + ggB[i,PB_k] A[i,PA_k])
 *   gA2[i,PA_k] += C_k ggB[i,PB_k] gO[i,PO_k];  gB2[i,PB_k] += C_k ggA[i,PA_k] gO[i,PO_k]
 * ggA / ggB may be NULL (their terms vanish); each output may be NULL (skipped). */
void FN(oracle_sap_vjp_vjp)(T *ggO, T *gA2, T *gB2, const T *ggA, const T *ggB, const T *gO,
                            const T *A, const T *B, const T *C, const int32_t *PA,
                            const int32_t *PB, const int32_t *PO, int64_t I, int64_t nA,
                            int64_t nB, int64_t nO, int64_t K) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < I; i++) {
        if (ggO) for (int64_t n = 0; n < nO; n++) ggO[i * nO + n] = 0;
        if (gA2) for (int64_t n = 0; n < nA; n++) gA2[i * nA + n] = 0;
        if (gB2) for (int64_t n = 0; n < nB; n++) gB2[i * nB + n] = 0;
        for (int64_t k = 0; k < K; k++) {
            T a = A[i * nA + PA[k]], b = B[i * nB + PB[k]], go = gO[i * nO + PO[k]];
            if (ggA) {
                T g = ggA[i * nA + PA[k]];
                if (ggO) ggO[i * nO + PO[k]] += g * b * C[k];
                if (gB2) gB2[i * nB + PB[k]] += g * go * C[k];
            }
            if (ggB) {
                T g = ggB[i * nB + PB[k]];
                if (ggO) ggO[i * nO + PO[k]] += g * a * C[k];
                if (gA2) gA2[i * nA + PA[k]] += g * go * C[k];
            }
        }
    }
}

/* O[P[j],k,l] += A[j,k]*B[j,l]; rows with no entry stay zero.  mops/src/opsa/cpu.tpp:31-52
 * Entries are visited in ascending j, as the reference's write list does; any index order
 * is accepted (the reference CPU code does not require sorted indices). */
void FN(oracle_opsa)(T *O, const T *A, const T *B, const int32_t *P, int64_t J, int64_t K,
                     int64_t L, int64_t nO) {
    for (int64_t x = 0; x < nO * K * L; x++) O[x] = 0;
    for (int64_t j = 0; j < J; j++) {
        T *o = O + (int64_t)P[j] * K * L;
        for (int64_t k = 0; k < K; k++)
            for (int64_t l = 0; l < L; l++) o[k * L + l] += A[j * K + k] * B[j * L + l];
    }
}

/* gA[j,k] = sum_l gO[P[j],k,l] B[j,l];  gB[j,l] = sum_k gO[P[j],k,l] A[j,k]
 * mops/src/opsa/cpu.tpp:89-110 */
void FN(oracle_opsa_vjp)(T *gA, T *gB, const T *gO, const T *A, const T *B, const int32_t *P,
                         int64_t J, int64_t K, int64_t L, int64_t nO) {
    (void)nO;
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < J; j++) {
        const T *g = gO + (int64_t)P[j] * K * L;
        if (gA)
            for (int64_t k = 0; k < K; k++) {
                T s = 0;
                for (int64_t l = 0; l < L; l++) s += g[k * L + l] * B[j * L + l];
                gA[j * K + k] = s;
            }
        if (gB)
            for (int64_t l = 0; l < L; l++) {
                T s = 0;
                for (int64_t k = 0; k < K; k++) s += g[k * L + l] * A[j * K + k];
                gB[j * L + l] = s;
            }
    }
}

/* Second-order terms of OPSA.  mops/src/opsa/cpu.tpp:114-246
 *   ggO[P_j,k,l] += ggA[j,k] B[j,l] + A[j,k] ggB[j,l]
 *   gA2[j,k] = sum_l gO[P_j,k,l] ggB[j,l];   gB2[j,l] = sum_k gO[P_j,k,l] ggA[j,k]
 * ggA / ggB may be NULL (their terms vanish); each output may be NULL (skipped). */
void FN(oracle_opsa_vjp_vjp)(T *ggO, T *gA2, T *gB2, const T *ggA, const T *ggB, const T *gO,
                             const T *A, const T *B, const int32_t *P, int64_t J, int64_t K,
                             int64_t L, int64_t nO) {
    if (ggO) for (int64_t x = 0; x < nO * K * L; x++) ggO[x] = 0;
    for (int64_t j = 0; j < J; j++) {
        const T *g = gO + (int64_t)P[j] * K * L;
        T *o = ggO ? ggO + (int64_t)P[j] * K * L : 0;
        if (gA2) for (int64_t k = 0; k < K; k++) gA2[j * K + k] = 0;
        if (gB2) for (int64_t l = 0; l < L; l++) gB2[j * L + l] = 0;
        if (ggA)
            for (int64_t k = 0; k < K; k++)
                for (int64_t l = 0; l < L; l++) {
                    if (o) o[k * L + l] += ggA[j * K + k] * B[j * L + l];
                    if (gB2) gB2[j * L + l] += ggA[j * K + k] * g[k * L + l];
                }
        if (ggB)
            for (int64_t k = 0; k < K; k++)
                for (int64_t l = 0; l < L; l++) {
                    if (o) o[k * L + l] += ggB[j * L + l] * A[j * K + k];
                    if (gA2) gA2[j * K + k] += ggB[j * L + l] * g[k * L + l];
                }
    }
}

/* O[PO[e],k,l] += A[e,k]*B[e,l]*W[PW[e],l]       mops/src/opsaw/cpu.tpp:35-53 */
void FN(oracle_opsaw)(T *O, const T *A, const T *B, const T *W, const int32_t *PW,
                      const int32_t *PO, int64_t E, int64_t K, int64_t L, int64_t nO) {
    for (int64_t x = 0; x < nO * K * L; x++) O[x] = 0;
    for (int64_t e = 0; e < E; e++) {
        T *o = O + (int64_t)PO[e] * K * L;
        const T *w = W + (int64_t)PW[e] * L;
        for (int64_t k = 0; k < K; k++)
            for (int64_t l = 0; l < L; l++) o[k * L + l] += A[e * K + k] * B[e * L + l] * w[l];
    }
}

/* gA[e,k] += gO[PO_e,k,l] B[e,l] W[PW_e,l];  gB[e,l] += gO[PO_e,k,l] A[e,k] W[PW_e,l];
 * gW[PW_e,l] += gO[PO_e,k,l] A[e,k] B[e,l]       mops/src/opsaw/cpu.tpp:77-129
 * gW sums run over entries in ascending e for each W row, as the reference's write list
 * over indices_W does. */
void FN(oracle_opsaw_vjp)(T *gA, T *gB, T *gW, const T *gO, const T *A, const T *B,
                          const T *W, const int32_t *PW, const int32_t *PO, int64_t E,
                          int64_t K, int64_t L, int64_t nO) {
    if (gA) for (int64_t x = 0; x < E * K; x++) gA[x] = 0;
    if (gB) for (int64_t x = 0; x < E * L; x++) gB[x] = 0;
    if (gW) for (int64_t x = 0; x < nO * L; x++) gW[x] = 0;
    for (int64_t e = 0; e < E; e++) {
        const T *g = gO + (int64_t)PO[e] * K * L;
        const T *w = W + (int64_t)PW[e] * L;
        for (int64_t k = 0; k < K; k++)
            for (int64_t l = 0; l < L; l++) {
                T go = g[k * L + l], a = A[e * K + k];
                if (gA) gA[e * K + k] += go * B[e * L + l] * w[l];
                if (gB) gB[e * L + l] += go * a * w[l];
                if (gW) gW[(int64_t)PW[e] * L + l] += go * a * B[e * L + l];
            }
    }
}

/* O[I_e, M3_n, b] += C_n A[e,M1_n] B[e,b] W[J_e, M2_n, b]    mops/src/sasaw/cpu.tpp:47-71
 * Argument names follow the C API: indices_A = M1, indices_W_1 = J, indices_W_2 = M2,
 * indices_output_1 = I, indices_output_2 = M3. */
void FN(oracle_sasaw)(T *O, const T *A, const T *B, const T *C, const T *W,
                      const int32_t *M1, const int32_t *Jw, const int32_t *M2,
                      const int32_t *Io, const int32_t *M3, int64_t E, int64_t nA, int64_t L,
                      int64_t N, int64_t nW0, int64_t nW1, int64_t nO1) {
    for (int64_t x = 0; x < nW0 * nO1 * L; x++) O[x] = 0;
    for (int64_t e = 0; e < E; e++) {
        T *o = O + (int64_t)Io[e] * nO1 * L;
        const T *w = W + (int64_t)Jw[e] * nW1 * L;
        for (int64_t n = 0; n < N; n++) {
            T ac = C[n] * A[e * nA + M1[n]];
            for (int64_t b = 0; b < L; b++)
                o[M3[n] * L + b] += ac * B[e * L + b] * w[M2[n] * L + b];
        }
    }
}

/* VJP of the above w.r.t. A, B and W.              mops/src/sasaw/cpu.tpp:99-168 */
void FN(oracle_sasaw_vjp)(T *gA, T *gB, T *gW, const T *gO, const T *A, const T *B,
                          const T *C, const T *W, const int32_t *M1, const int32_t *Jw,
                          const int32_t *M2, const int32_t *Io, const int32_t *M3, int64_t E,
                          int64_t nA, int64_t L, int64_t N, int64_t nW0, int64_t nW1,
                          int64_t nO1) {
    if (gA) for (int64_t x = 0; x < E * nA; x++) gA[x] = 0;
    if (gB) for (int64_t x = 0; x < E * L; x++) gB[x] = 0;
    if (gW) for (int64_t x = 0; x < nW0 * nW1 * L; x++) gW[x] = 0;
    for (int64_t e = 0; e < E; e++) {
        const T *g = gO + (int64_t)Io[e] * nO1 * L;
        const T *w = W + (int64_t)Jw[e] * nW1 * L;
        T *gw = gW ? gW + (int64_t)Jw[e] * nW1 * L : 0;
        for (int64_t n = 0; n < N; n++) {
            T c = C[n], ac = c * A[e * nA + M1[n]];
            for (int64_t b = 0; b < L; b++) {
                T go = g[M3[n] * L + b];
                if (gA) gA[e * nA + M1[n]] += go * c * B[e * L + b] * w[M2[n] * L + b];
                if (gB) gB[e * L + b] += go * ac * w[M2[n] * L + b];
                if (gw) gw[M2[n] * L + b] += go * ac * B[e * L + b];
            }
        }
    }
}
