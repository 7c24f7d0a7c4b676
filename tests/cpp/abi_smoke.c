/* The header is plain C and the library links from C: what a cgo / hsc2hs / JNI stub relies on.
 * Makes no compute call; on a machine without a driver accb_init reports ACCB_ENODRIVER. */
#include <stdio.h>
#include <string.h>

#include "accb200.h"

int main(void) {
    accb_array a;
    accb_value_type t;
    InputArray in;
    OutputArray out;
    memset(&a, 0, sizeof a);
    memset(&t, 0, sizeof t);
    memset(&in, 0, sizeof in);
    memset(&out, 0, sizeof out);
    a.rank = 1;
    a.shape[0] = 4;
    t.comp_bytes[0] = 4;
    if (sizeof(in) != 2 * sizeof(void *) || sizeof(out) != 3 * sizeof(void *)) return 2;
    if (!accb_version() || !accb_version()[0]) return 3;
    {
        int st = accb_init();
        accb_group *grp = NULL;
        int devs[2] = {0, 0};
        if (st != ACCB_OK && st != ACCB_ENODRIVER && st != ACCB_ECUDA) return 4;
        if (st != ACCB_OK) {
            /* every entry point fails with a status and a message instead of crashing */
            if (accb_group_create(devs, 2, &grp) == ACCB_OK || grp != NULL) return 5;
            if (!accb_last_error(NULL) || !accb_last_error(NULL)[0]) return 6;
            if (accelerateCreate(0, NULL) != NULL) return 7;
            /* the AccFFI.h spelling: argc / argv are accepted and ignored */
            if (accelerateInit(0, NULL, 0, NULL) != NULL) return 8;
        }
    }
    puts("OK");
    return 0;
}
