/*
 * Drop-in replacement for the reference's openai_blocksparse.h, which holds a second copy of
 * bst_sgemm_nt (openai_blocksparse.h:202-233).  The function lives in blocksparse.h here.
 */
#ifndef SFB_DROPIN_OPENAI_BLOCKSPARSE_H
#define SFB_DROPIN_OPENAI_BLOCKSPARSE_H
#include "blocksparse.h"
#endif
