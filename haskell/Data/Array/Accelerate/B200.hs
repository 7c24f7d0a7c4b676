{-# LANGUAGE BangPatterns #-}
-- |
-- Module      : Data.Array.Accelerate.B200
-- Description : Run Accelerate programs on NVIDIA B200 GPUs through libaccb200.so
--
-- NOT COMPILED HERE: the build machine of this repository has no GHC.
--
-- The interface of "Data.Array.Accelerate.CUDA" (accelerate-cuda,
-- Data/Array/Accelerate/CUDA.hs:184-200,232-353): a program written against
-- that module changes its import and nothing else.
--
-- > import Data.Array.Accelerate        as A
-- > import Data.Array.Accelerate.B200   as B200
-- >
-- > dotp :: Vector Float -> Vector Float -> Scalar Float
-- > dotp xs ys = B200.run $ A.fold (+) 0 (A.zipWith (*) (use xs) (use ys))
--
-- What differs underneath: the program is translated once into an op list of
-- the library ("Data.Array.Accelerate.B200.Execute") whose nodes name skeleton
-- kernels instantiated with the user's scalar functions
-- ("Data.Array.Accelerate.B200.CodeGen"); running it on host arrays is ONE
-- foreign call, which uploads, launches and downloads -- in pieces, so that
-- the host link and the GPU overlap, where the program allows it.
--
module Data.Array.Accelerate.B200 (

  Arrays,

  -- * Synchronous execution
  run, run1, stream, runWith, run1With, streamWith,

  -- * Asynchronous execution
  Async, wait, poll, cancel,
  runAsync, run1Async, runAsyncWith, run1AsyncWith,

  -- * Execution contexts
  Context, create, destroy, defaultContext,

  -- * Memory
  performGC, performGCWith,

) where

import Control.Concurrent.Async                         ( Async, asyncBound, wait, poll, cancel )
import System.IO.Unsafe

import Data.Array.Accelerate.Array.Sugar                ( Arrays )
import Data.Array.Accelerate.Smart                      ( Acc )
import Data.Array.Accelerate.Trafo

import Data.Array.Accelerate.B200.Context
import Data.Array.Accelerate.B200.Execute


-- | Compile and run a complete embedded array program on device 0.
-- It is recommended to use 'run1' whenever the same program is applied to
-- different data.
run :: Arrays a => Acc a -> a
run = runWith defaultContext

-- | As 'run', in the given execution context (CUDA.hs:248-251).
runWith :: Arrays a => Context -> Acc a -> a
runWith ctx a = unsafePerformIO $ wait =<< runAsyncWith ctx a

runAsync :: Arrays a => Acc a -> IO (Async a)
runAsync = runAsyncWith defaultContext

-- | The front end's sharing recovery and fusion run here exactly as for the
-- reference (convertAccWith, CUDA.hs:271); the delayed term then goes to
-- 'compileAcc' of this backend.
runAsyncWith :: Arrays a => Context -> Acc a -> IO (Async a)
runAsyncWith ctx a = asyncBound $ do
  let !acc = convertAccWith config a
  prog <- compileAcc ctx acc
  r    <- executeAcc prog
  destroyProgram prog
  return r

-- | Prepare an array function once and apply it many times: the returned
-- closure goes straight to the execution phase (CUDA.hs:307-330).
run1 :: (Arrays a, Arrays b) => (Acc a -> Acc b) -> a -> b
run1 = run1With defaultContext

run1With :: (Arrays a, Arrays b) => Context -> (Acc a -> Acc b) -> a -> b
run1With ctx f =
  let go = run1AsyncWith ctx f
  in \a -> unsafePerformIO $ wait =<< go a

run1Async :: (Arrays a, Arrays b) => (Acc a -> Acc b) -> a -> IO (Async b)
run1Async = run1AsyncWith defaultContext

run1AsyncWith :: (Arrays a, Arrays b) => Context -> (Acc a -> Acc b) -> a -> IO (Async b)
run1AsyncWith ctx f = \a -> asyncBound (executeAfun1 afun a)
  where
    !acc  = convertAfunWith config f
    !afun = unsafePerformIO (compileAfun1 ctx acc)      -- once; kernels come from the library's cache afterwards

-- | Apply one compiled function to a lazily read list of inputs (CUDA.hs:333-347).
stream :: (Arrays a, Arrays b) => (Acc a -> Acc b) -> [a] -> [b]
stream = streamWith defaultContext

streamWith :: (Arrays a, Arrays b) => Context -> (Acc a -> Acc b) -> [a] -> [b]
streamWith ctx f = map go
  where
    !go = run1With ctx f

-- | Evict every device array that has a host copy (CUDA.hs:433-441).
performGC :: IO ()
performGC = performGCWith defaultContext

-- What the front end is asked to do: the same phases the reference asks for
-- (CUDA.hs:356-366), with fusion on -- a fused producer becomes the functor of
-- the consuming skeleton.
config :: Phase
config = Phase
  { recoverAccSharing      = True
  , recoverExpSharing      = True
  , recoverSeqSharing      = True
  , floatOutAccFromExp     = True
  , enableAccFusion        = True
  , convertOffsetOfSegment = True      -- foldSeg receives offsets, not lengths (CUDA/Execute.hs:320-324)
  }
