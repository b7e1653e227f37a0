/* A C caller of the host-side entry points of libqk_kernels.so (no GPU needed): what a
 * compiled host such as the reference's server links against.  Exit code 0 = all checks
 * passed; each failure prints the line it came from. */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "qk_kernels.h"

static int failures = 0;
#define CHECK(cond)                                                      \
    do {                                                                 \
        if (!(cond)) {                                                   \
            fprintf(stderr, "%s:%d: %s\n", __FILE__, __LINE__, #cond);   \
            ++failures;                                                  \
        }                                                                \
    } while (0)

int main(void) {
    /* pack_bits: element 8j+k of a row at bit k of byte j, +1 -> 1 (core.rs:129-162) */
    const int8_t factor[2 * 10] = {1, -1, 1, 1, -1, -1, -1, 1, 1, -1,
                                   -1, -1, -1, -1, -1, -1, -1, -1, -1, 1};
    uint8_t packed[4] = {0xAA, 0xAA, 0xAA, 0xAA};
    CHECK(qk_pack_bits(factor, 20, 2, 10, packed, 4) == QK_OK);
    CHECK(packed[0] == 0x8D && packed[1] == 0x01 && packed[2] == 0x00 && packed[3] == 0x02);
    int8_t back[20];
    CHECK(qk_unpack_bits(packed, 4, 2, 10, back, 20) == QK_OK);
    CHECK(memcmp(back, factor, 20) == 0);

    /* refusals carry the reference's texts (parity.rs:1062-1081) */
    const int8_t bad[2] = {1, 3};
    uint8_t one[1];
    CHECK(qk_pack_bits(bad, 2, 1, 2, one, 1) == QK_ERR_VALUE);
    CHECK(strcmp(qk_last_error(),
                 "pack_bits expects values in {-1, +1}; got 3 at row 0, column 1") == 0);
    size_t words = 0;
    CHECK(qk_validate_packed(7, 2, 10, &words) == QK_ERR_VALUE);
    CHECK(strcmp(qk_last_error(), "packed length 7 does not match 2 rows x 2 bitplanes") == 0);
    CHECK(qk_validate_packed(4, 2, 10, &words) == QK_OK && words == 2);

    /* dtype tags (dtype.rs:99-129) */
    int32_t tag = -1;
    CHECK(qk_dtype_from_name("bfloat16", &tag) == QK_OK && tag == 2);
    CHECK(strcmp(qk_dtype_name(1), "float32") == 0);
    CHECK(qk_dtype_from_name("float16", &tag) == QK_ERR_VALUE);

    /* sign_estimate (core.rs:193-197) */
    const double xs[4] = {0.5, -0.0, -2.0, 0.0};
    int8_t sg[4];
    CHECK(qk_sign_estimate(xs, 4, sg) == QK_OK);
    CHECK(sg[0] == 1 && sg[1] == 1 && sg[2] == -1 && sg[3] == 1);

    /* joint_itq (core.rs:327-424): deterministic in the seed, +-1 outputs, refusals */
    double u_hat[6 * 2], v_hat[4 * 2];
    for (int i = 0; i < 12; ++i) u_hat[i] = (double)((i * 7) % 5) - 2.0 + 0.125 * i;
    for (int i = 0; i < 8; ++i) v_hat[i] = (double)((i * 3) % 4) - 1.5 - 0.0625 * i;
    int8_t u1[12], v1[8], u2[12], v2[8];
    size_t it1 = 0, it2 = 0;
    int32_t c1 = -1, c2 = -1;
    CHECK(qk_joint_itq(u_hat, 12, v_hat, 8, 6, 4, 2, 50, 1e-12, 42, u1, v1, &it1, &c1) == QK_OK);
    CHECK(qk_joint_itq(u_hat, 12, v_hat, 8, 6, 4, 2, 50, 1e-12, 42, u2, v2, &it2, &c2) == QK_OK);
    CHECK(memcmp(u1, u2, 12) == 0 && memcmp(v1, v2, 8) == 0 && it1 == it2 && c1 == c2);
    CHECK(it1 >= 1 && it1 <= 50 && (c1 == 0 || c1 == 1));
    for (int i = 0; i < 12; ++i) CHECK(u1[i] == 1 || u1[i] == -1);
    CHECK(qk_joint_itq(u_hat, 12, v_hat, 8, 6, 4, 0, 50, 1e-12, 42, u1, v1, &it1, &c1) ==
          QK_ERR_VALUE);
    CHECK(strcmp(qk_last_error(), "joint_itq expects non-empty factors") == 0);

    /* a qpk1 stream that is too short is refused, not read */
    const uint8_t junk[8] = {'Q', 'P', 'K', '1', 2, 0, 0, 0};
    qk_qpk1_info info;
    CHECK(qk_qpk1_parse(junk, 8, &info) == QK_ERR_VALUE);

    /* no device in this process: the typed init failure names the hint */
    CHECK(strlen(qk_gpu_init_hint()) > 20);
    CHECK(strlen(qk_backend_version()) > 0);

    if (failures) return 1;
    puts("host ABI ok");
    return 0;
}
