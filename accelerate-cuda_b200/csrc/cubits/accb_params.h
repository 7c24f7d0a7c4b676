/*
 * accb_params.h -- the one argument block every skeleton kernel receives.
 *
 * Shared by the host runtime (plain C++) and the device code, so it is plain
 * C.  It plays the role of the generated parameter lists of accelerate-cuda
 * (environment arrays first, then the skeleton's own arguments:
 * Data/Array/Accelerate/CUDA/CodeGen/Base.hs:344-383 and
 * Data/Array/Accelerate/CUDA/Execute.hs:938-951), but with a fixed layout so
 * that the host can marshal arguments for a functor it knows nothing about.
 *
 * Arrays of tuples are structure-of-arrays: one pointer ("slot") per
 * flattened scalar component (Base.hs:69-79).  Shapes are stored innermost
 * extent first: shape[0] is the fastest-varying dimension.
 */
#ifndef ACCB_PARAMS_H
#define ACCB_PARAMS_H

#define ACCB_MAX_IN 16   /* input component slots (all environment arrays together) */
#define ACCB_MAX_OUT 8   /* output component slots */
#define ACCB_MAX_ARR 8   /* environment arrays */
#define ACCB_MAX_RANK 4
#define ACCB_MAX_AUX 6
#define ACCB_MAX_IP 12
#define ACCB_SCALAR_BYTES 64
#define ACCB_FOLD_DEFER_MAX 1024 /* segments one foldSeg launch can hand over to its second launch (below) */

/* accb_kparams.flags */
#define ACCB_F_VEC 1u        /* every slot is 16-byte aligned: 128-bit path allowed */
#define ACCB_F_HAS_SEED 2u   /* scalars[0..] hold the seed value(s) */
#define ACCB_F_INCLUSIVE 4u  /* scan: inclusive result */
#define ACCB_F_RIGHT 8u      /* scan: right-to-left */
#define ACCB_F_SEED_PTR 16u  /* scalars[0..8) is a device pointer to the seed */
#define ACCB_F_CARRY 32u     /* foldAll: aux[2] points to the result of the part of the array before this one */

typedef struct accb_kparams {
    const void *in[ACCB_MAX_IN];
    void *out[ACCB_MAX_OUT];
    void *aux[ACCB_MAX_AUX];        /* skeleton-private: scratch, status words, totals, locks */
    long long n;                    /* problem size in elements (source size for permute) */
    long long ip[ACCB_MAX_IP];      /* skeleton-private integers */
    int in_shape[ACCB_MAX_ARR][ACCB_MAX_RANK];
    int in_first[ACCB_MAX_ARR];     /* first slot of each environment array */
    int out_shape[ACCB_MAX_RANK];
    unsigned int flags;
    int pad_;
    long long base;                 /* index of this launch's first element in the whole array: what the functor
                                       is told is base + position (a launch may cover a piece of a larger array) */
    unsigned char scalars[ACCB_SCALAR_BYTES]; /* user scalars, packed in declaration order */
} accb_kparams;


/* Segments far longer than the rest would keep one thread, warp or block of a foldSeg kernel busy long after the
 * others are done.  Such a segment is put on this list instead (runtime-owned scratch, zero between launches) and
 * a second launch reduces the listed segments with all blocks. */
typedef struct accb_deferred_segments {
    unsigned int count;    /* segments put on the list (may exceed the capacity: the excess was not deferred) */
    unsigned int finished; /* blocks of the second launch that are done; the last one clears the list */
    long long unit[ACCB_FOLD_DEFER_MAX];        /* row * segments + segment */
    unsigned int arrived[ACCB_FOLD_DEFER_MAX];  /* pieces of a listed segment reduced so far */
} accb_deferred_segments;

#endif
